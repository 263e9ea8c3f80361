"""``bench.py --impl reference``: run the unmodified reference engine on the benchmark config.

The reference serves Qwen3.5-style checkpoints only through its native plane, the ``pocketllm_engine``
executable (cpp_engine/engine/main.cpp).  ``baseline/_ref/bin/pocketllm_engine`` is that executable built
from the untouched sources with CMake for sm_100 against NCCL and cuBLAS; ``baseline/_ref`` also holds the
pip-installed Python packages.  This module writes the same synthetic checkpoint our own arm uses (same
seeded generator, the reference's tensor names, safetensors + config.json), starts one engine process per
rank in the reference's persistent-stdin mode (``--qwen-persistent-stdin``, main.cpp:656-764), sends
``warmup + steps`` requests and reports the timings the engine itself prints
(``qwen_persistent_result=1 ... prefill_tokens_per_s= ... decode_tokens_per_s=``).

None of this repository's kernels or runtime is on that path; only the checkpoint writer is shared.
"""
from __future__ import annotations

import os
import re
import shutil
import subprocess
import queue
import sys
import tempfile
import threading
import time

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
EXE = os.path.join(REF, "bin", "pocketllm_engine")

PUBLISHED_PREFILL_TPS = 1811.1
PUBLISHED_DECODE_TPS = 37.12


def _unavailable(why: str) -> dict:
    return {"impl": "reference", "unavailable": why}


def _scratch_root() -> str:
    for root in ("/dev/shm", tempfile.gettempdir()):
        try:
            st = shutil.disk_usage(root)
            if st.free > 40 << 30:
                return root
        except OSError:
            continue
    return tempfile.gettempdir()


def write_checkpoint(cfg, directory: str, device) -> float:
    """Synthetic checkpoint in the reference's naming; returns seconds spent."""
    from deepseek_v4_2080ti_b200.formats import safetensors_io
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh

    t0 = time.time()
    safetensors_io.write_checkpoint(directory, qh.synth_state(cfg, 0, device), shard_bytes=2 << 30,
                                    config_json=cfg.to_json())
    return time.time() - t0


def _field(line: str, key: str) -> float:
    m = re.search(rf"\b{key}=([0-9.eE+-]+)", line)
    return float(m.group(1)) if m else float("nan")


def drive_engine(cmd, env, line: str, *, leader: bool, warmup: int, steps: int, budget: float, t_arm0: float) -> dict:
    """Run one engine process in persistent-stdin mode under a wall-clock budget (seconds, counted from ``t_arm0``).

    The leader feeds one request line at a time and waits for its ``qwen_persistent_result=1`` line, so it can stop
    between requests when the budget runs low and still report what completed.  The first request doubles as
    warm-up (the engine has no JIT or graph capture); the other warm-up requests asked for are sent only when all of
    ``warmup + steps`` fit the budget, judged from the engine's own wall time of the first request.  Follower ranks
    take their commands from the leader over the reference's own channel: they get their output drained and a bound
    on their lifetime."""
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            env=env)
    t_start = time.time()
    lines: "queue.Queue[str | None]" = queue.Queue()
    tail: list[str] = []

    def _reader():
        for out in proc.stdout:
            lines.put(out)
        lines.put(None)

    threading.Thread(target=_reader, daemon=True).start()

    def left() -> float:
        return budget - (time.time() - t_arm0)

    def next_result(limit: float):
        """The next result line, None if the engine exited or ``limit`` seconds passed."""
        t_end = time.time() + limit
        while True:
            try:
                out = lines.get(timeout=max(0.05, t_end - time.time()))
            except queue.Empty:
                return None
            if out is None:
                return None
            tail.append(out.rstrip()[:300])
            del tail[:-8]
            if out.startswith("qwen_persistent_result=1"):
                return out

    def finish(grace: float) -> int:
        try:
            proc.stdin.close()
        except (BrokenPipeError, OSError):
            pass
        try:
            return proc.wait(timeout=grace)
        except subprocess.TimeoutExpired:
            proc.kill()
            return proc.wait()

    if not leader:
        while proc.poll() is None and left() + 90 > 0:
            next_result(5.0)
        return {"rc": finish(10)}

    results, req_wall = [], []
    want_warm = max(1, warmup)
    warm_done = None
    why_short = ""
    while True:
        if warm_done is None and results:
            per = _field(results[0], "wall") * 1.15     # the first host wall also holds the weight load
            warm_done = want_warm if left() // per >= (want_warm - 1) + steps else 1
        if len(results) >= (warm_done or 1) + steps:
            break
        if results and left() < max([_field(results[0], "wall")] + req_wall[1:]) * 1.15:
            why_short = f"time budget of {int(budget)} s"
            break
        t_req = time.time()
        try:
            proc.stdin.write(line)
            proc.stdin.flush()
        except (BrokenPipeError, OSError):
            why_short = "engine closed its input"
            break
        out = next_result(max(30.0, left()))
        if out is None:
            try:                                        # end of output can be seen a moment before the process is gone
                proc.wait(timeout=1.0)
            except subprocess.TimeoutExpired:
                pass
            why_short = ("engine exited" if proc.poll() is not None
                         else f"time budget of {int(budget)} s (request in flight)")
            break
        results.append(out)
        req_wall.append(time.time() - t_req)
    t_done = time.time()
    return {"results": results, "req_wall": req_wall, "warm_done": warm_done or 1, "why_short": why_short,
            "rc": finish(30), "tail": tail, "t_start": t_start, "t_done": t_done, "t_arm0": t_arm0}


def run(args) -> dict:
    if not os.path.isfile(EXE):
        return _unavailable("baseline/_ref/bin/pocketllm_engine is not installed (CMake build of the reference's cpp_engine missing)")
    import torch

    if not torch.cuda.is_available():
        return _unavailable("no GPU visible")
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    cfg = qh.QwenHybridConfig.config2() if args.layers == 64 else qh.QwenHybridConfig(num_hidden_layers=args.layers)
    if getattr(args, "tiny", False):
        cfg = qh.QwenHybridConfig.tiny(layers=4)
    tag = os.environ.get("MASTER_PORT", "0")
    work = os.path.join(_scratch_root(), f"pocketllm_ref_{tag}_{cfg.num_hidden_layers}l_{cfg.hidden_size}h")
    ready = os.path.join(work, "READY")
    ckpt_s = 0.0
    if rank == 0:
        if not os.path.exists(ready):
            shutil.rmtree(work, ignore_errors=True)
            os.makedirs(work, exist_ok=True)
            torch.cuda.set_device(local)
            ckpt_s = write_checkpoint(cfg, work, torch.device("cuda", local))
            torch.cuda.empty_cache()
            open(ready, "w").write("ok")
    else:
        t0 = time.time()
        while not os.path.exists(ready):
            if time.time() - t0 > 1800:
                return _unavailable("timed out waiting for rank 0 to write the synthetic checkpoint")
            time.sleep(0.5)

    ctx = args.prompt + args.decode + 64
    id_path = os.path.join(work, f"nccl_id_{os.getpid() if world == 1 else tag}")
    # --smoke-layers: the executable runs ONE layer unless told otherwise (main.cpp:35); ask for all of them
    cmd = [EXE, "--ckpt", work, "--smoke-forward", "--smoke-layers", str(cfg.num_hidden_layers),
           "--qwen-persistent-stdin", "--max-context", str(ctx),
           "--qwen-no-prefix-cache", "--prefill-chunk-tokens", str(args.chunk), "--tp-world", str(world),
           "--tp-rank", str(rank), "--device", str(local)]
    if world > 1:
        cmd += ["--nccl-id-path", id_path]
    env = dict(os.environ)
    env.setdefault("NCCL_DEBUG", "WARN")
    gen = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=gen, dtype=torch.int32).tolist()
    line = f"{args.decode} " + " ".join(map(str, prompt)) + "\n"
    budget = float(os.environ.get("POCKETLLM_REFERENCE_BUDGET_S", "480"))
    run_ = drive_engine(cmd, env, line, leader=(rank == 0), warmup=args.warmup, steps=args.steps,
                        budget=budget, t_arm0=time.time() - ckpt_s)
    if rank != 0:
        return {}
    shutil.rmtree(work, ignore_errors=True)
    results, req_wall, warm_done, why_short = run_["results"], run_["req_wall"], run_["warm_done"], run_["why_short"]
    t_start, t_done, t_arm0 = run_["t_start"], run_["t_done"], run_["t_arm0"]
    timed = results[warm_done:]
    if not timed:
        return _unavailable(f"reference engine completed {len(results)} request(s) at tp{world} ({why_short}; "
                            f"rc={run_['rc']}): " + " | ".join(t[:200] for t in run_["tail"][-3:]))
    eng_wall = [_field(r, "wall") for r in results]
    pre_s = [_field(r, "prefill_seconds") for r in timed]
    dec_s = [_field(r, "decode_seconds") for r in timed]
    pre = sum(pre_s) / len(pre_s)
    dec = sum(dec_s) / len(dec_s)
    prefill_tps = args.prompt / pre
    decode_tps = (args.decode - 1) / dec
    m = re.search(r"(?<![a-z_])tokens=([0-9,]+)", timed[-1])
    toks = m.group(1).split(",") if m else []
    return {
        "impl": "reference", "metric": "prefill_tok_s", "value": round(prefill_tps, 1), "unit": "tok/s",
        "n_gpus": world, "steps": len(timed), "warmup": warm_done, "steps_asked": args.steps,
        "warmup_asked": args.warmup, "truncated": why_short or None, "ms_per_step": round((pre + dec) * 1e3, 3),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": round(prefill_tps / PUBLISHED_PREFILL_TPS, 2),
        "dtype": "fp16", "data": "synthetic (random-init FP8 block-128 weights, random token ids)",
        "prefill_ms": round(pre * 1e3, 3), "decode_tok_s": round(decode_tps, 2),
        "decode_ms_per_token": round(dec * 1e3 / (args.decode - 1), 4),
        "decode_vs_baseline": round(decode_tps / PUBLISHED_DECODE_TPS, 2),
        "config": {"model": f"Qwen3.8-27B-FP8-shaped hybrid ({cfg.num_hidden_layers}L, hidden {cfg.hidden_size}, vocab {cfg.vocab_size})",
                   "global_batch": 1, "seq_len": args.prompt, "decode_tokens": args.decode,
                   "parallelism": f"tp{world}", "weights": "fp8_e4m3_block128",
                   "path": "pocketllm_engine --qwen-persistent-stdin (timings printed by the engine, host clock around synchronous calls)"},
        "e2e": {"value": round(prefill_tps, 1), "unit": "tok/s",
                "what": "the engine's own request path: token ids in over stdin, H2D inside prefill, next token read back",
                "h2d_bytes_per_step": args.prompt * 4, "d2h_bytes_per_step": 4 * args.decode},
        "wall_breakdown_s": {"checkpoint_write": round(ckpt_s, 1), "engine_start_to_first_request_done": round(
                                 (t_done - t_start) - sum(req_wall[1:]), 1),
                             "request_host_wall_mean": round(sum(req_wall) / len(req_wall), 2),
                             "request_engine_wall_mean": round(sum(eng_wall) / len(eng_wall), 2),
                             "requests_done": len(results), "total": round(time.time() - t_arm0, 1)},
        "first_tokens": [int(t) for t in toks[:16]],
    }
