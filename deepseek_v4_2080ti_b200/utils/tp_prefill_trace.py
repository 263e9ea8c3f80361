"""Per-kernel device-time table of ONE tensor-parallel prefill, taken on rank 0 with the activity tracer of
``torch.profiler`` (kernel begin / end records; launches are not serialised or replayed, so kernels that wait for a
peer's flags show the time they spent waiting).  Run it one process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        -m deepseek_v4_2080ti_b200.utils.tp_prefill_trace --prompt 8192 [--layers 64] [--out trace.json]

The figures are shares of a traced step; the benchmark's own numbers come from CUDA events without a tracer.  With
many short kernels per rank the tracer's per-launch cost is not small (at 8 ranks the traced 27B-shaped prefill took
177 ms against 96 ms plain: the host falls behind, ranks drift apart and the flag waits inside the GEMMs grow), so read
the table for which kernels wait, not for absolute times.  Prints, for rank 0: the step's wall on the device, the busy time of the main stream, and
the kernels grouped by name with launches, total and mean microseconds.  The reference has phase timers around its
prefill loop for the same purpose (cpp_engine/engine/qwen_engine.cpp: the ``ar.*`` / ``gemm.*`` counters)."""
from __future__ import annotations

import argparse
import json
import re
import sys


def _short(name: str) -> str:
    name = name.replace("(anonymous namespace)::", "").replace("<unnamed>::", "")
    name = re.sub(r"^void\s+", "", name)
    name = re.sub(r"\(.*$", "", name)
    return name[:90]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=64)
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--out", default="")
    args = ap.parse_args()

    import torch
    import torch.distributed as dist
    from torch.profiler import ProfilerActivity, profile

    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.parallel import tp

    rank, world, local = tp.init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = qh.QwenHybridConfig.config2() if args.layers == 64 else qh.QwenHybridConfig(num_hidden_layers=args.layers)
    comm = tp.PeerComm(slot_elems=args.chunk * cfg.hidden_size) if world > 1 else None
    weights = qh.QwenHybridWeights(cfg, qh.synth_state(cfg, 0, dev), dev, rank, world)
    max_ctx = args.prompt + 64
    rt = qh.QwenHybridRuntime(cfg, weights, max_slots=2, max_context=max_ctx, comm=comm)
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=torch.Generator().manual_seed(1),
                           dtype=torch.int32).to(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def step():
        slot = rt.allocate()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        rt.prefill(slot, prompt, args.chunk)
        e1.record()
        torch.cuda.synchronize()
        rt.free(slot)
        return e0.elapsed_time(e1)

    plain = 0.0
    for _ in range(args.warmup):
        barrier()
        plain = step()
    if comm is not None:
        comm.check()
    barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        traced = step()
    barrier()
    if rank == 0:
        rows: dict[str, list[float]] = {}
        spans = []
        for e in prof.events():
            if getattr(e, "device_type", None) is None or "CUDA" not in str(e.device_type):
                continue
            dur = float(e.time_range.end - e.time_range.start)
            if dur <= 0.0 or e.name.startswith("Memcpy") or e.name.startswith("Memset"):
                continue
            rows.setdefault(_short(e.name), []).append(dur)
            spans.append((e.time_range.start, e.time_range.end))
        total = sum(sum(v) for v in rows.values())
        # union of the kernel intervals: time during which at least one kernel was running
        spans.sort()
        busy, cur_s, cur_e = 0.0, None, None
        for s, t in spans:
            if cur_e is None or s > cur_e:
                if cur_e is not None:
                    busy += cur_e - cur_s
                cur_s, cur_e = s, t
            else:
                cur_e = max(cur_e, t)
        if cur_e is not None:
            busy += cur_e - cur_s
        table = sorted(((k, len(v), sum(v)) for k, v in rows.items()), key=lambda r: -r[2])
        rec = {"world": world, "prompt": args.prompt, "layers": cfg.num_hidden_layers, "prefill_ms_plain": round(plain, 3),
               "prefill_ms_traced": round(traced, 3), "kernel_time_sum_ms": round(total / 1e3, 3),
               "any_kernel_running_ms": round(busy / 1e3, 3),
               "kernels": [{"name": k, "launches": n, "total_us": round(t, 1), "mean_us": round(t / n, 2),
                            "share_of_step": round(t / 1e3 / traced, 4)} for k, n, t in table[:40]]}
        print(f"world {world}: prefill {plain:.2f} ms plain, {traced:.2f} ms traced; kernel time summed {total / 1e3:.2f} ms, "
              f"some kernel running {busy / 1e3:.2f} ms")
        for k, n, t in table[:40]:
            print(f"  {t / 1e3:9.3f} ms  {n:5d} x {t / n:9.2f} us  {100 * t / 1e3 / traced:5.1f}%  {k}")
        if args.out:
            with open(args.out, "w") as f:
                json.dump(rec, f, indent=1)
    barrier()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
    sys.exit(0)
