#!/usr/bin/env python
"""Headline benchmark: prefill and decode tokens/s of the Qwen3.8-27B-FP8-shaped hybrid model
(64 layers, hidden 5120, 48 Gated-DeltaNet + 16 gated-GQA layers, FP8 E4M3 128x128 block-scaled
weights, bf16 activations) with synthetic random-init weights and random-token prompts.

One step = one request: prefill of ``--prompt`` tokens, then ``--decode`` greedy tokens at batch 1
over the paged KV cache (+ an optional batch-32 decode phase reported separately).  Phases are
device-timed with CUDA events, max over ranks; ``value`` is prefill tokens/s (the reference's
headline number, docs/benchmarking.md:21-32 convention: first generated token belongs to prefill).

  python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]
N > 1 is launched by ``python -m torch.distributed.run --nproc-per-node N`` (tensor parallel over NCCL/NVLink).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

PUBLISHED_PREFILL_TPS = 1811.1   # reference, 8,192-token prompt, 4x RTX 2080 Ti (cpp_engine/include/qwen_engine.hpp:54-55)
PUBLISHED_DECODE_TPS = 37.12     # reference, batch-1 decode, same hardware (docs/models/qwen3.8-27b-fp8.md:71)


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--prompt", type=int, default=8192)
    ap.add_argument("--decode", type=int, default=256)
    ap.add_argument("--batch-decode", type=int, default=32, help="extra batched decode phase (0 = skip)")
    ap.add_argument("--layers", type=int, default=64, help="debug only; the reported config is 64")
    ap.add_argument("--chunk", type=int, default=8192)
    ap.add_argument("--tiny", action="store_true", help="debug only: 4-layer hidden-256 model")
    ap.add_argument("--spec", choices=["none", "mtp", "ngram"], default="none",
                    help="config 2: also run greedy speculative decoding after the timed steps (mtp: a random-init "
                         "multi-token-prediction head is added to the synthetic checkpoint) and report acceptance")
    ap.add_argument("--spec-tokens", type=int, default=2)
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="benchmark configuration: 2 Qwen-shaped FP8 hybrid (the headline, default), 3 MiniMax-shaped "
                         "GGUF GQA-MoE, 4 DeepSeek-V4-Flash-shaped MLA + indexer + FP4 MoE, 5 GLM-shaped GGUF DSA-MoE")
    from deepseek_v4_2080ti_b200.utils import model_bench
    model_bench.add_arguments(ap, layers=False)
    args = ap.parse_args()
    args.prompt_given = "--prompt" in sys.argv
    return args


# configs 3-5: published numbers of the reference on 4x RTX 2080 Ti for the models these shapes follow
MOE_CONFIGS = {
    3: ("gqa_moe", 107.0, 10.32, "MiniMax-M2.7 UD-IQ1_M 256-token prefill / 43-layer decode (docs/models/minimax-m2.7.md:46-48)"),
    4: ("dsv4", 402.0, 3.7, "DeepSeek-V4-Flash C++ FP4 prefill @ 32,768 / decode (docs/models/deepseek-v4.md:52-54)"),
    5: ("glm", 0.79, 0.66, "GLM-5.2 UD-Q2_K_XL prefill / decode (docs/models/glm-5.2.md:51-52)"),
}


def run_moe_config(args) -> None:
    """Configs 3-5 through utils/model_bench.py: same timing rules and JSON keys as the headline config."""
    import torch
    import torch.distributed as dist

    from deepseek_v4_2080ti_b200.parallel import tp
    from deepseek_v4_2080ti_b200.utils import model_bench
    from deepseek_v4_2080ti_b200.utils.clocks import ClockSampler

    family, pub_prefill, pub_decode, pub_src = MOE_CONFIGS[args.config]
    d_prompt, d_decode, d_chunk, d_pp = model_bench.FAMILY_DEFAULTS[family]
    args.family = family
    args.layers = 0 if args.layers == 64 else args.layers        # 64 is the headline config's own default: all layers
    if not args.prompt_given:
        args.prompt = d_prompt
    args.decode = min(args.decode, d_decode)
    args.chunk = min(args.chunk, d_chunk)
    if args.config == 5 and args.pp == 1 and args.gpus >= 2 and os.environ.get("B200_BENCH_GLM_PP", "0") == "1":
        args.pp = d_pp
    if args.impl == "reference":
        why = {3: "the installed reference's GGUF path does not import: `python -m src.cli.generate_gguf` on a synthetic "
                  "minimax-m2 GGUF fails in src/components/moe/registry.py:12 with ModuleNotFoundError: No module named "
                  "'src.models.glm_dsa' (the reference's setup.py does not list that package, so pip does not install it)",
               5: "the installed reference has no src.models.glm_dsa package (absent from the reference's setup.py package "
                  "list), so `python -m src.cli.generate_glm` cannot be imported from baseline/_ref",
               4: "the reference's DeepSeek-V4 is a different architecture from this configuration (single KV head of "
                  "dim 512 + window + learned compressor, not MLA q_lora 1024 / kv_lora 512 with a top-2048 indexer): "
                  "none of its engines can load a checkpoint of this shape"}[args.config]
        print(json.dumps({"impl": "reference", "config": args.config, "unavailable": why}), flush=True)
        return
    rank, world, local = tp.init_distributed()
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    rec = model_bench.run_family(args, rank, world, dev, steps=args.steps, warmup=args.warmup,
                                 clock_sampler=lambda: ClockSampler(local))
    if rec is not None:
        out = {"metric": "prefill_tok_s", "value": rec["prefill_tok_s"], "unit": "tok/s", "n_gpus": world,
               "steps": rec["steps"], "warmup": rec["warmup"],
               "ms_per_step": round(rec["prefill_ms"] + rec["decode_ms_per_token"] * args.decode, 3),
               "higher_is_better": True, "scaling": "strong", "vs_baseline": round(rec["prefill_tok_s"] / pub_prefill, 2),
               "dtype": "bf16", "data": rec["data"], "impl": "b200", "prefill_ms": rec["prefill_ms"],
               "decode_tok_s": rec["decode_tok_s"], "decode_ms_per_token": rec["decode_ms_per_token"],
               "decode_vs_baseline": round(rec["decode_tok_s"] / pub_decode, 2), "baseline_source": pub_src,
               "config": {"model": rec["model"], "global_batch": 1, "seq_len": args.prompt, "decode_tokens": args.decode,
                          "parallelism": rec["parallelism"], "collectives": rec["collectives"],
                          "weights_gb_per_rank": rec["weights_gb_per_rank"],
                          "l2_policy": "inputs larger than L2: every step streams the rank's weight set"},
               "clocks": rec.get("clocks"), "gpu_launches": rec.get("gpu_launches_eager"),
               "detail": {k: v for k, v in rec.items() if k.startswith("mtp_") or k in ("plain_total_ms", "launches_per_decode_step", "gpu_launches_eager",
                                                                                     "build_seconds", "timing")}}
        print(json.dumps(out), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args) -> None:
    from baseline import reference_arm
    rec = reference_arm.run(args)
    if rec:   # ranks other than 0 of a multi-rank run return nothing
        print(json.dumps(rec), flush=True)


def main() -> None:
    args = parse()
    if args.config != 2:
        run_moe_config(args)
        return
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist

    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.ops import _lib
    from deepseek_v4_2080ti_b200.parallel import tp
    from deepseek_v4_2080ti_b200.utils.clocks import ClockSampler

    rank, world, local = tp.init_distributed()
    assert world == args.gpus or world == 1, (world, args.gpus)
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cfg = qh.QwenHybridConfig.config2()
    if args.tiny:
        cfg = qh.QwenHybridConfig.tiny(layers=4)
    elif args.layers != 64:
        cfg = qh.QwenHybridConfig(num_hidden_layers=args.layers)
    comm = None
    if world > 1:
        # peer-memory collectives: row-parallel GEMMs reduce in their epilogue (one-shot pushes at 2 ranks and for decode
        # batches, owner-reduces two-shot beyond); the slot holds one whole prefill chunk of hidden states
        comm = tp.PeerComm(slot_elems=args.chunk * cfg.hidden_size)
    bdec = args.batch_decode
    max_slots = max(1, bdec) + 1
    t0 = time.time()
    state = qh.synth_state(cfg, 0, dev)
    if args.spec == "mtp":
        import itertools
        from deepseek_v4_2080ti_b200.models.reference_cpu.qwen_hybrid_ref import synth_mtp_state
        state = itertools.chain(state, ((n, t.to(dev)) for n, t in synth_mtp_state(cfg, 0, std=0.02, fp8_linears=True)))
    weights = qh.QwenHybridWeights(cfg, state, dev, rank, world)
    max_ctx = args.prompt + args.decode + 64
    rt = qh.QwenHybridRuntime(cfg, weights, max_slots=max_slots, max_context=max_ctx, comm=comm,
                              num_blocks=((max_ctx + 63) // 64) * 2 + max_slots * 8 + 2)
    torch.cuda.synchronize()
    if rank == 0:
        print(f"[bench] weights {weights.nbytes() / 1e9:.2f} GB/rank built in {time.time() - t0:.1f}s", file=sys.stderr)

    gen = torch.Generator().manual_seed(1)
    prompt_host = torch.randint(0, cfg.vocab_size, (args.prompt,), generator=gen, dtype=torch.int32)
    prompt_dev = prompt_host.to(dev)
    prompt_list = prompt_host.tolist()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    ev = lambda: torch.cuda.Event(enable_timing=True)

    def device_request():
        """Kernel-only timing: inputs already on the device, tokens fed back on the device, nothing read by the
        host inside the timed region.  Returns (prefill_ms, decode_ms, launches)."""
        slot = rt.allocate()
        e0, e1, e2 = ev(), ev(), ev()
        e0.record()
        tok = rt.prefill(slot, prompt_dev, args.chunk)
        e1.record()
        launches = rt.launches
        for _ in range(args.decode - 1):
            tok = rt.decode([slot], tok.to(torch.int32))
            launches += rt.launches
        e2.record()
        torch.cuda.synchronize()
        rt.free(slot)
        return e0.elapsed_time(e1), e1.elapsed_time(e2), launches

    # ---- end-to-end arm: the public API (pocketllm.LLM over the engine backend) on the same runtime.  Every request
    # carries its prompt as host token ids (copied to the device from pinned memory inside the call) and every
    # generated token is read back to the host.
    from pocketllm import LLM, SamplingParams
    from pocketllm.api.types import EngineArgs
    from pocketllm.backends.native_backend import NativeBackend
    from deepseek_v4_2080ti_b200.runtime.loader import RuntimeAdapter

    llm = LLM(backend=NativeBackend(EngineArgs(model="synthetic:bench", max_model_len=max_ctx,
                                                prefill_chunk_tokens=args.chunk, tensor_parallel_size=1),
                                    runtime=RuntimeAdapter(rt, max_ctx)))
    sp = SamplingParams(max_tokens=args.decode, temperature=0.0)

    def api_request():
        res = llm.generate([{"prompt_token_ids": prompt_list}], sp)[0]
        return res.timings.prefill_seconds * 1e3, res.timings.decode_seconds * 1e3, len(res.token_ids)

    def batch_decode_phase(steps: int):
        """bdec sequences with short prompts decoding together; returns ms per step."""
        slots = [rt.allocate() for _ in range(bdec)]
        firsts = []
        for i, s in enumerate(slots):
            p = torch.randint(0, cfg.vocab_size, (64,), generator=gen, dtype=torch.int32).to(dev)
            firsts.append(rt.prefill(s, p))
        cur = torch.cat(firsts).to(torch.int32)
        for _ in range(3):
            cur = rt.decode(slots, cur).to(torch.int32).clone()
        barrier()
        e0, e1 = ev(), ev()
        e0.record()
        for _ in range(steps):
            cur = rt.decode(slots, cur).to(torch.int32).clone()
        e1.record()
        torch.cuda.synchronize()
        for s in slots:
            rt.free(s)
        return e0.elapsed_time(e1) / steps

    fallback = False
    for i in range(args.warmup):
        device_request()
        if i == 0:
            # A kernel that gave up on a wait (a peer that never signalled) shows here, after one request, not after
            # the whole run has crawled through its wait budgets.  All ranks agree on the outcome; if any saw an
            # error, the group re-synchronises and the rest of the run uses the library collectives.
            bad = int(_lib.status_word(dev).item())
            if world > 1:
                tb = torch.tensor([bad], device=dev, dtype=torch.int32)
                dist.all_reduce(tb, op=dist.ReduceOp.MAX)
                bad = int(tb.item())
            if bad:
                if comm is None:
                    _lib.check_status()
                print(f"[bench] rank {rank}: a device wait expired (status {bad}); continuing on the NCCL path",
                      file=sys.stderr, flush=True)
                comm.recover(degrade=True)
                rt._graphs.clear()
                fallback = True
                device_request()
                _lib.check_status()
    api_request()
    barrier()
    pre_ms, dec_ms, launches = [], [], 0
    api_pre, api_dec = [], []
    with ClockSampler(local) as clk:
        barrier()
        for _ in range(args.steps):
            p, d, l = device_request()
            pre_ms.append(p)
            dec_ms.append(d)
            launches += l
        barrier()
        w0 = time.time()
        for _ in range(args.steps):
            p, d, n = api_request()
            assert n == args.decode, n
            api_pre.append(p)
            api_dec.append(d)
        barrier()
        wall = time.time() - w0
        bd_ms = batch_decode_phase(64) if bdec > 0 else None
    spec_rec = None
    if args.spec != "none":
        # outside the timed region and the clock sampling: greedy speculative decoding of the same request
        from deepseek_v4_2080ti_b200.models.qwen_spec import QwenSpeculator
        sp_ = QwenSpeculator(rt, k=args.spec_tokens, method=args.spec)
        sp_.generate(prompt_dev, min(args.decode, 16), args.chunk)          # warm-up
        sp_.stats = type(sp_.stats)()
        barrier()
        e0, e1, e2 = ev(), ev(), ev()
        slot = sp_.allocate()
        e0.record()
        out_tokens = [sp_.prefill(slot, prompt_dev, args.chunk)]
        e1.record()
        while len(out_tokens) < args.decode:
            out_tokens.extend(sp_.step(slot))
        e2.record()
        torch.cuda.synchronize()
        sp_.free(slot)
        spec_rec = {"method": args.spec, "draft_tokens": args.spec_tokens, "accept_rate": round(sp_.stats.accept_rate, 4),
                    "tokens_per_pass": round(sp_.stats.tokens_per_pass, 3),
                    "decode_tok_s": round((len(out_tokens) - 1) / (e1.elapsed_time(e2) / 1e3), 2),
                    "note": "random-init weights: the draft head is untrained, so acceptance is chance level"}
    _lib.check_status()
    clocks = clk.summary()

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    mean = lambda v: sum(v) / len(v)
    pre = max_over_ranks(mean(pre_ms))
    dec = max_over_ranks(mean(dec_ms))
    e_pre = max_over_ranks(mean(api_pre))
    e_dec = max_over_ranks(mean(api_dec))
    wall_step = max_over_ranks(wall / args.steps * 1e3)
    prefill_tps = args.prompt / (pre / 1e3)
    decode_tps = (args.decode - 1) / (dec / 1e3)
    if rank == 0:
        model = "Qwen3.8-27B-FP8-shaped hybrid (64L, hidden 5120, 48 GDN + 16 gated GQA, vocab 151936)"
        if args.tiny or args.layers != 64:
            model = f"DEBUG {cfg.num_hidden_layers} layers hidden {cfg.hidden_size}"
        rec = {
            "metric": "prefill_tok_s", "value": round(prefill_tps, 1), "unit": "tok/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(pre + dec, 3),
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(prefill_tps / PUBLISHED_PREFILL_TPS, 2), "dtype": "bf16",
            "data": "synthetic (random-init FP8 block-128 weights, random token ids)", "impl": "b200",
            "prefill_ms": round(pre, 3), "decode_tok_s": round(decode_tps, 2),
            "decode_ms_per_token": round(dec / (args.decode - 1), 4),
            "decode_vs_baseline": round(decode_tps / PUBLISHED_DECODE_TPS, 2),
            "config": {"model": model, "global_batch": 1, "seq_len": args.prompt, "decode_tokens": args.decode,
                       "parallelism": f"tp{world}", "weights": "fp8_e4m3_block128", "kv_cache": "bf16 paged (block 64)",
                       "l2_policy": "inputs larger than L2: every step streams the full weight set (>= 3 GB/rank)"},
            "e2e": {"value": round(args.prompt / (e_pre / 1e3), 1), "unit": "tok/s",
                    "decode_tok_s": round((args.decode - 1) / (e_dec / 1e3), 2),
                    "what": "pocketllm.LLM.generate on host token ids: list -> pinned tensor -> H2D inside the call, "
                            "every generated token read back (D2H) before the next decode step; host clock",
                    "h2d_bytes_per_step": int(prompt_host.numel() * 4 + (args.decode - 1) * 4),
                    "d2h_bytes_per_step": 4 * args.decode, "wall_ms_per_step": round(wall_step, 3)},
            "gpu_launches": int(launches),
            "clocks": clocks,
        }
        if bd_ms is not None:
            bd = max_over_ranks(bd_ms)
            rec["decode_batch"] = {"batch": bdec, "ms_per_step": round(bd, 4), "tok_s": round(bdec / (bd / 1e3), 1)}
        if spec_rec is not None:
            rec["speculative"] = spec_rec
        if comm is not None:
            # fused = kernels that carry their collective (reduce-scatter / all-gather GEMMs, the reduce + norm + gather
            # kernel, GEMM + all-reduce epilogues); standalone = peer-memory collectives launched on their own
            rec["collective_fallback"] = fallback
            rec["fused_collective_calls"] = int(comm.fused_calls)
            rec["standalone_peer_collectives"] = int(comm.standalone_calls)
            rec["config"]["prefill_collectives"] = ("sequence-parallel: GEMM->reduce-scatter, reduce+norm+all-gather, "
                                                    "all-gather->GEMM over peer memory") \
                if comm.sp_rows(min(args.chunk, args.prompt), cfg.hidden_size) else "GEMM + all-reduce"
        print(json.dumps(rec), flush=True)
    elif bd_ms is not None:
        max_over_ranks(bd_ms)
    if world > 1:
        comm.close()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
