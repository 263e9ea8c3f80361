"""Single-kernel micro-benchmarks (CUDA-event timed, L2 flushed between iterations).

  python -m deepseek_v4_2080ti_b200.utils.microbench gemm --t 8192 --n 5120 --k 5120 [--fmt fp8|bf16] [--splits S]
  python -m deepseek_v4_2080ti_b200.utils.microbench attn_prefill --t 8192 --hq 40 --hkv 8
  python -m deepseek_v4_2080ti_b200.utils.microbench gdn --t 8192 --hv 32 --hk 16
  python -m deepseek_v4_2080ti_b200.utils.microbench swiglu --t 4096 --n 17408 --k 5120     # n = I: gate_up GEMM [2I, K] + SwiGLU

Used for roofline numbers and as the small-case command for ncu captures (``--iters 1 --warmup 1``).
"""
from __future__ import annotations

import argparse
import json

import torch


def _flush(buf):
    buf.zero_()


def timeit(fn, iters, warmup, flush=True):
    buf = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            _flush(buf)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    times.sort()
    return times[len(times) // 2], times[0]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "swiglu", "attn_prefill", "attn_decode", "gdn", "gdn_step"])
    ap.add_argument("--t", type=int, default=8192)
    ap.add_argument("--n", type=int, default=5120)
    ap.add_argument("--k", type=int, default=5120)
    ap.add_argument("--fmt", default="fp8")
    ap.add_argument("--splits", type=int, default=None)
    ap.add_argument("--kernel", default="auto", choices=["auto", "decode_warps", "stream", "stream_presplit"],
                    help="gemm: which kernel serves small T (stream_presplit times the GEMM without the activation split)")
    ap.add_argument("--hq", type=int, default=40)
    ap.add_argument("--hkv", type=int, default=8)
    ap.add_argument("--hv", type=int, default=32)
    ap.add_argument("--hk", type=int, default=16)
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    a = ap.parse_args()
    from ..formats import fp8 as fp8fmt
    from ..ops import _lib, attention, gdn, gemm
    torch.manual_seed(0)
    rec = {"op": a.op}
    if a.op == "gemm":
        w = torch.randn(a.n, a.k, device="cuda") * 0.05
        x = torch.randn(a.t, a.k, device="cuda").bfloat16()
        if a.fmt == "fp8":
            q, s = fp8fmt.quantize_block128(w)
            pl = gemm.PackedLinear.from_fp8(q, s)
        else:
            pl = gemm.PackedLinear.from_bf16(w.bfloat16())
        del w
        out = torch.empty(a.t, a.n, dtype=torch.bfloat16, device="cuda")
        if a.kernel == "stream_presplit":
            xs = gemm.split_activations(x)
            fn = lambda: gemm.linear_stream(x, pl, out=out, splits=a.splits, xsplit=xs)
        else:
            st = {"auto": None, "decode_warps": False, "stream": True}[a.kernel]
            fn = lambda: gemm.linear(x, pl, out=out, splits=a.splits, stream=st)
        med, best = timeit(fn, a.iters, a.warmup)
        flops = 2.0 * a.t * a.n * a.k
        byts = pl.nbytes() + x.numel() * 2 + out.numel() * 2
        rec.update(t=a.t, n=a.n, k=a.k, fmt=a.fmt, kernel=a.kernel, ms=med, ms_best=best, tflops=flops / med / 1e9, gbs=byts / med / 1e6)
    elif a.op == "swiglu":
        # feed-forward first half: x [T, K] x [gate | up] [2I, K] -> silu(gate) * up [T, I]; fused epilogue against
        # GEMM + silu_mul.  The FP8 -> bf16 expansion is inside both timings (it runs on every prefill call).
        from ..ops import basic
        w = torch.randn(2 * a.n, a.k, device="cuda") * 0.05
        q, s = fp8fmt.quantize_block128(w)
        pl = gemm.PackedLinear.from_fp8(q, s)
        del w
        x = torch.randn(a.t, a.k, device="cuda").bfloat16()
        out = torch.empty(a.t, a.n, dtype=torch.bfloat16, device="cuda")
        assert gemm.swiglu_fusable(a.t, pl), "shape not taken by the fused kernel"
        fused, fbest = timeit(lambda: gemm.linear_swiglu(x, pl, out=out), a.iters, a.warmup)
        gu = torch.empty(a.t, 2 * a.n, dtype=torch.bfloat16, device="cuda")
        plain, pbest = timeit(lambda: basic.silu_mul(gemm.linear(x, pl, out=gu)), a.iters, a.warmup)
        flops = 4.0 * a.t * a.n * a.k
        rec.update(t=a.t, inter=a.n, k=a.k, ms=fused, ms_best=fbest, tflops=flops / fused / 1e9, ms_unfused=plain,
                   ms_unfused_best=pbest, tflops_unfused=flops / plain / 1e9)
    elif a.op == "attn_prefill":
        bs = 64
        nb = (a.ctx + bs - 1) // bs
        q = torch.randn(a.t, a.hq, 128, device="cuda").bfloat16()
        kc = torch.randn(nb + 1, a.hkv, bs, 128, device="cuda").bfloat16()
        vc = torch.randn(nb + 1, a.hkv, bs, 128, device="cuda").bfloat16()
        bt = torch.arange(1, nb + 1, dtype=torch.int32, device="cuda")[None].contiguous()
        i32 = lambda v: torch.tensor([v], dtype=torch.int32, device="cuda")
        qs, ql, kl = i32(0), i32(a.t), i32(a.ctx)
        fn = lambda: attention.prefill(q, kc, vc, bt, qs, ql, kl, a.t)
        med, best = timeit(fn, a.iters, a.warmup)
        # causal: query i sees ctx - t + i + 1 keys
        pairs = a.t * (a.ctx - a.t) + a.t * (a.t + 1) / 2
        flops = 4.0 * pairs * 128 * a.hq
        rec.update(t=a.t, ctx=a.ctx, hq=a.hq, hkv=a.hkv, ms=med, ms_best=best, tflops=flops / med / 1e9)
    elif a.op == "attn_decode":
        bs = 64
        nbs = (a.ctx + bs - 1) // bs
        q = torch.randn(a.batch, a.hq, 128, device="cuda").bfloat16()
        kc = torch.randn(nbs * a.batch + 1, a.hkv, bs, 128, device="cuda").bfloat16()
        vc = torch.randn(nbs * a.batch + 1, a.hkv, bs, 128, device="cuda").bfloat16()
        bt = (torch.arange(nbs * a.batch, dtype=torch.int32, device="cuda") + 1).view(a.batch, nbs).contiguous()
        kl = torch.full((a.batch,), a.ctx, dtype=torch.int32, device="cuda")
        fn = lambda: attention.decode(q, kc, vc, bt, kl, max_kv_len=a.ctx)
        med, best = timeit(fn, a.iters, a.warmup)
        byts = 2.0 * a.batch * a.ctx * a.hkv * 128 * 2
        rec.update(batch=a.batch, ctx=a.ctx, ms=med, ms_best=best, gbs=byts / med / 1e6)
    elif a.op == "gdn":
        ld = 2 * a.hk * 128 + a.hv * 128
        mixed = torch.randn(a.t, ld, device="cuda").bfloat16()
        g = -torch.rand(a.t, a.hv, device="cuda") * 0.5
        beta = torch.rand(a.t, a.hv, device="cuda")
        state = torch.zeros(a.hv, 128, 128, device="cuda")
        fn = lambda: gdn.chunked(mixed, 0, a.hk * 128, 2 * a.hk * 128, g, beta, state, a.hv, a.hk)
        med, best = timeit(fn, a.iters, a.warmup)
        rec.update(t=a.t, hv=a.hv, hk=a.hk, ms=med, ms_best=best, tok_per_s=a.t / med * 1e3)
    elif a.op == "gdn_step":
        ld = 2 * a.hk * 128 + a.hv * 128
        mixed = torch.randn(a.batch, ld, device="cuda").bfloat16()
        g = -torch.rand(a.batch, a.hv, device="cuda") * 0.5
        beta = torch.rand(a.batch, a.hv, device="cuda")
        states = torch.zeros(a.batch, a.hv, 128, 128, device="cuda")
        slots = torch.arange(a.batch, dtype=torch.int32, device="cuda")
        fn = lambda: gdn.step(states, slots, mixed, 0, a.hk * 128, 2 * a.hk * 128, g, beta, a.hv, a.hk)
        med, best = timeit(fn, a.iters, a.warmup)
        byts = 2.0 * states.numel() * 4
        rec.update(batch=a.batch, ms=med, ms_best=best, gbs=byts / med / 1e6)
    torch.cuda.synchronize()
    _lib.check_status()
    print(json.dumps(rec), flush=True)


if __name__ == "__main__":
    main()
