"""Prefill / decode throughput of the MoE families on synthetic checkpoints of the benchmark shapes.

    # MiniMax-M2.7-shaped GGUF model, attention TP8 + experts EP8
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29533 \\
        -m deepseek_v4_2080ti_b200.utils.model_bench --family gqa_moe --prompt 4096 --decode 256
    # GLM-5.2-shaped GGUF mix as a 2-stage layer pipeline with TP4/EP4 per stage
    ... -m deepseek_v4_2080ti_b200.utils.model_bench --family glm --pp 2 --prompt 2048 --decode 256
    # DeepSeek-V4-Flash-shaped MLA + indexer + FP4 experts, TP8 + EP8, MTP depth-1 drafting
    ... -m deepseek_v4_2080ti_b200.utils.model_bench --family dsv4 --prompt 32768 --decode 256 --mtp

Timing: CUDA events around the prefill and around the decode loop, after one untimed warm-up request, max over ranks.
Weights are random-init in the checkpoint formats; ``--expert-pool P`` draws P distinct experts per layer and repeats
them (the quantisers dominate start-up otherwise); ``--layers N`` runs the first N layers only and says so in the
output (a reduced run is a kernel-level probe, not a model number).  One JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import time

import torch
import torch.distributed as dist

from ..parallel import pp as pplib
from ..parallel import tp


def _timed(fn):
    torch.cuda.synchronize()
    if dist.is_initialized():
        dist.barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    out = fn()
    b.record()
    torch.cuda.synchronize()
    ms = torch.tensor([a.elapsed_time(b)], device="cuda")
    if dist.is_initialized():
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return out, float(ms.item())


def _gqa_moe(args, rank, world, dev):
    from ..models import gqa_moe as gm
    cfg = gm.GqaMoeConfig.config3()
    if args.layers:
        cfg = dataclasses.replace(cfg, n_layers=args.layers)
    t0 = time.time()
    store = gm.TensorStore(gm.synth_tensors(cfg, seed=0, device=dev, expert_pool=args.expert_pool))
    w = gm.GqaMoeGpuWeights(cfg, store, dev, rank, world)
    del store
    torch.cuda.empty_cache()
    comm = None
    if world > 1:
        comm = tp.TPComm() if args.nccl else tp.PeerComm(slot_elems=max(1 << 20, args.chunk * cfg.hidden))
    rt = gm.GqaMoeRuntime(cfg, w, max_slots=1, max_context=args.prompt + args.decode + 64, comm=comm)
    build_s = time.time() - t0
    prompt = torch.randint(0, cfg.vocab, (args.prompt,), generator=torch.Generator().manual_seed(1), dtype=torch.int32).to(dev)

    def request(n_decode, prompt=prompt):
        slot = rt.allocate()
        tok, pre_ms = _timed(lambda: rt.prefill(slot, prompt, args.chunk))

        def loop():
            t = tok
            for _ in range(n_decode):
                t = rt.decode([slot], t.to(torch.int32))
            return t
        _, dec_ms = _timed(loop)
        rt.free(slot)
        return pre_ms, dec_ms

    warm = lambda: request(4, prompt[:args.chunk])     # one full chunk (workspaces, lazy kernel set-up, graphs)
    run = lambda: request(args.decode)
    desc = {"model": f"MiniMax-M2.7-shaped GQA-MoE GGUF ({cfg.n_layers}L of 62, hidden {cfg.hidden}, {cfg.n_experts} experts top-{cfg.top_k}, "
                     f"attn {cfg.attn_type}, experts {cfg.gate_up_type}/{cfg.down_type})",
            "parallelism": f"tp{world}+ep{world}", "collectives": "nccl" if args.nccl else "peer-memory kernels",
            "hidden": cfg.hidden, "launches": lambda: rt.launches}
    return warm, run, w.nbytes(), build_s, desc


def _mla(args, rank, world, dev, glm: bool):
    from ..models import mla_moe as mm
    from ..models import mla_moe_gpu as mg
    cfg = mm.MlaMoeConfig.glm_5_2_shaped() if glm else mm.MlaMoeConfig.deepseek_v4_flash_shaped()
    if args.mtp and not glm:
        cfg = dataclasses.replace(cfg, mtp_layers=1)
    if args.layers:
        cfg = dataclasses.replace(cfg, num_layers=args.layers, first_dense_layers=min(cfg.first_dense_layers, args.layers))
    stages = max(1, args.pp)
    layout = pplib.PipelineLayout(rank, world, stages)
    link = pplib.PipelineLink(layout, dev) if stages > 1 else None
    lo, hi = pplib.split_layers(cfg.num_layers, stages)[layout.stage]
    tpw, tpr = layout.tp, layout.tp_rank
    per = cfg.num_experts // tpw
    t0 = time.time()
    routed_tp = bool(getattr(args, "routed_tp", False)) and tpw > 1
    state = mm.synth_state(cfg, 0, dev, expert_range=(0, cfg.num_experts) if routed_tp else (tpr * per, (tpr + 1) * per),
                           expert_pool=args.expert_pool, layer_range=(lo, hi))
    w = mg.MlaMoeGpuWeights(cfg, state, dev, rank=tpr, world=tpw, layer_range=(lo, hi),
                            routed_tp=True if getattr(args, "routed_tp", False) else None,
                            gguf_mix=mg.GLM_GGUF_MIX if glm else None, dense_fp8=not glm)
    torch.cuda.empty_cache()
    comm = None
    if tpw > 1:
        group = link.stage_group if link is not None else None
        comm = tp.TPComm(group) if (args.nccl or stages > 1) else tp.PeerComm(slot_elems=max(1 << 20, args.chunk * cfg.hidden_size))
    rt = mg.MlaMoeGpuRuntime(cfg, w, max_context=args.prompt + 2 * args.decode + 64, comm=comm, pipeline=link)
    build_s = time.time() - t0
    prompt = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=torch.Generator().manual_seed(1), dtype=torch.int32).to(dev)
    from ..ops import basic
    last = layout.is_last

    def request(n_decode, mtp, prompt=prompt):
        rt.reset()
        if mtp:
            out, total_ms = _timed(lambda: rt.generate_mtp(prompt, n_decode + 1, chunk=args.chunk))
            return None, total_ms

        def prefill():
            logits = None
            for s in range(0, prompt.numel(), args.chunk):
                o = rt.forward(prompt[s:s + args.chunk])
                logits = o[-1:] if o is not None else None
            tok = basic.argmax(logits) if last else None
            return link.share_token(tok) if link is not None else tok
        tok, pre_ms = _timed(prefill)

        graph = link is None and not args.eager_decode
        if graph:                                      # capture the step of this context bucket outside the timed loop
            rt.decode_step(tok.to(torch.int32))
            rt.length -= 1                             # the row is written again by the first timed step

        def loop():
            t = tok
            for _ in range(n_decode):
                if graph:
                    t = rt.decode_step(t.to(torch.int32))
                    continue
                o = rt.forward(t.to(torch.int32))
                t = basic.argmax(o) if last else None
                if link is not None:
                    t = link.share_token(t)
            return t
        _, dec_ms = _timed(loop)
        if link is not None:
            link.drain()
        return pre_ms, dec_ms

    warm = lambda: request(2, False, prompt[:args.chunk])      # one full chunk
    run = lambda: request(args.decode, False)

    def extra_fn(pre_ms, dec_ms):
        if not (args.mtp and w.mtp):
            return {}
        _, spec_ms = request(args.decode, True)
        return {"mtp_total_ms": round(spec_ms, 2), "mtp_steps": rt.spec_stats["steps"],
                "mtp_accepted": rt.spec_stats["accepted"], "plain_total_ms": round(pre_ms + dec_ms, 2)}
    name = "GLM-5.2-shaped MLA + DSA indexer MoE, GGUF mix Q8_0/Q4_K/Q2_K/IQ3_XXS" if glm else \
        "DeepSeek-V4-Flash-shaped MLA + indexer MoE, FP8 dense + FP4 experts"
    desc = {"model": f"{name} ({cfg.num_layers}L of {78 if glm else 43}, hidden {cfg.hidden_size}, {cfg.num_experts} experts top-{cfg.experts_per_token}, "
                     f"index top-{cfg.index_topk})",
            "parallelism": (f"pp{stages} x " if stages > 1 else "") + f"tp{tpw}+ep{tpw}",
            "collectives": "nccl" if (args.nccl or stages > 1) else "peer-memory kernels", "hidden": cfg.hidden_size,
            "extra": extra_fn}
    nbytes = sum(t.numel() * t.element_size() for t in _tensors(w))
    return warm, run, nbytes, build_s, desc


def _tensors(obj, seen=None, depth=0):
    """Every tensor reachable from a weights object (for the resident-bytes figure)."""
    seen = set() if seen is None else seen
    if depth > 6 or id(obj) in seen:
        return
    if isinstance(obj, torch.Tensor):
        if obj.data_ptr() not in seen:
            seen.add(obj.data_ptr())
            yield obj
        return
    if isinstance(obj, (str, bytes, int, float, bool, type(None), torch.device, torch.dtype)):
        return
    seen.add(id(obj))
    if isinstance(obj, (list, tuple)):
        for x in obj:
            yield from _tensors(x, seen, depth + 1)
    elif isinstance(obj, dict):
        for x in obj.values():
            yield from _tensors(x, seen, depth + 1)
    elif hasattr(obj, "__dict__"):
        for x in vars(obj).values():
            yield from _tensors(x, seen, depth + 1)


FAMILY_DEFAULTS = {           # the benchmark shapes: (prompt, decode, chunk, pipeline stages)
    "gqa_moe": (4096, 256, 4096, 1), "dsv4": (32768, 256, 4096, 1), "glm": (2048, 256, 2048, 2),
}


def add_arguments(ap: argparse.ArgumentParser, layers: bool = True) -> None:
    if layers:
        ap.add_argument("--layers", type=int, default=0, help="run only the first N layers (reported as such)")
    ap.add_argument("--expert-pool", type=int, default=4)
    ap.add_argument("--pp", type=int, default=1, help="pipeline stages (glm / dsv4)")
    ap.add_argument("--routed-tp", action="store_true",
                    help="glm / dsv4: every rank holds all routed experts with 1/world of their width (GLM_ROUTED_TP=1)")
    ap.add_argument("--mtp", action="store_true", help="dsv4: also time depth-1 speculative decoding")
    ap.add_argument("--eager-decode", action="store_true", help="MLA families: launch every decode kernel instead of replaying a graph")
    ap.add_argument("--nccl", action="store_true", help="library collectives instead of the peer-memory kernels")


def run_family(args, rank: int, world: int, dev, steps: int = 1, warmup: int = 1, clock_sampler=None) -> dict | None:
    """Build the family's synthetic model, run ``warmup`` untimed and ``steps`` timed requests (prefill of
    ``args.prompt`` tokens + ``args.decode`` greedy tokens, CUDA events, max over ranks) and return the record
    (rank 0) or None.  ``clock_sampler``: a context-manager factory sampling the GPU clocks over the timed region."""
    import contextlib
    with torch.no_grad():
        build = _gqa_moe if args.family == "gqa_moe" else (lambda *a: _mla(*a, args.family == "glm"))
        warm, run, nbytes, build_s, desc = build(args, rank, world, dev)
        for _ in range(max(1, warmup)):
            warm()
        pre, dec = [], []
        from ..ops import _lib as _lib0
        launches0 = _lib0.LAUNCHES
        with (clock_sampler() if clock_sampler else contextlib.nullcontext()) as clk:
            for _ in range(max(1, steps)):
                p, d = run()
                pre.append(p)
                dec.append(d)
        eager_launches = _lib0.LAUNCHES - launches0
        pre_ms, dec_ms = sum(pre) / len(pre), sum(dec) / len(dec)
        extra = desc.pop("extra", None)
        launches = desc.pop("launches", None)
        more = extra(pre_ms, dec_ms) if extra else {}
    from ..ops import _lib
    _lib.check_status()
    if rank != 0:
        return None
    rec = {"family": args.family, "n_gpus": world, "prompt_tokens": args.prompt, "decode_tokens": args.decode,
           "steps": len(pre), "warmup": max(1, warmup),
           "prefill_ms": round(pre_ms, 2), "prefill_tok_s": round(args.prompt / pre_ms * 1e3, 1),
           "decode_ms_per_token": round(dec_ms / max(1, args.decode), 3),
           "decode_tok_s": round(args.decode / dec_ms * 1e3, 2), "weights_gb_per_rank": round(nbytes / 1e9, 2),
           "build_seconds": round(build_s, 1), "data": "synthetic random-init, expert pool %d" % args.expert_pool,
           "timing": "CUDA events, max over ranks, after a one-chunk warm-up request", **desc, **more}
    # kernels of this package launched from the host inside the timed region; kernels replayed inside a captured
    # decode graph are not in this count (launches_per_decode_step x decode tokens of them per request)
    rec["gpu_launches_eager"] = int(eager_launches)
    if launches:
        rec["launches_per_decode_step"] = launches()
    if clock_sampler and clk is not None:
        rec["clocks"] = clk.summary()
    return rec


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--family", choices=["gqa_moe", "glm", "dsv4"], required=True)
    ap.add_argument("--prompt", type=int, default=2048)
    ap.add_argument("--decode", type=int, default=64)
    ap.add_argument("--chunk", type=int, default=4096)
    ap.add_argument("--steps", type=int, default=1)
    ap.add_argument("--warmup", type=int, default=1)
    add_arguments(ap)
    args = ap.parse_args()
    rank, world, local = tp.init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    rec = run_family(args, rank, world, dev, args.steps, args.warmup)
    if rec is not None:
        print(json.dumps(rec), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
