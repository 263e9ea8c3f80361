"""Host dot-product micro-benchmark: weight bytes streamed per second by the CPU kernels of ``lib/libb200_cpu.so``
(raw GGUF Q8_0 / Q2_K / IQ2_XXS rows, INT8 W8A8 routed experts, FP4 routed experts).

    python -m deepseek_v4_2080ti_b200.utils.cpu_dot_bench [--rows 4096] [--cols 4096] [--threads 0] [--repeat 5]

Prints one JSON line per kernel: {"kernel", "ms", "weight_gbs", "threads"}; the best of ``repeat`` runs.
Reference counterpart: the int8 dot-product micro-benchmark src/csrc/dot_microbench.cpp."""
from __future__ import annotations

import argparse
import json
import time

import torch


def _best(fn, repeat: int) -> float:
    fn()
    best = float("inf")
    for _ in range(repeat):
        t0 = time.perf_counter()
        fn()
        best = min(best, time.perf_counter() - t0)
    return best


def run(rows: int = 4096, cols: int = 4096, threads: int = 0, repeat: int = 5) -> list[dict]:
    from ..formats.gguf import quant
    from ..formats.gguf.constants import GGMLType
    from ..models import mla_moe
    g = torch.Generator().manual_seed(0)
    x = torch.randn(1, cols, generator=g)
    out = []
    for name in ("Q8_0", "Q2_K", "IQ2_XXS"):
        t = GGMLType[name]
        raw = quant.quantize(torch.randn(min(rows, 256), cols, generator=g), t).repeat((rows + 255) // 256, 1)[:rows].contiguous()
        sec = _best(lambda: mla_moe.cpu_gguf_linear(x, raw, int(t), threads), repeat)
        out.append({"kernel": f"gguf_{name.lower()}_gemv", "ms": sec * 1e3, "weight_gbs": raw.numel() / sec / 1e9, "threads": threads})
    e, k, inter = 8, 2, max(32, rows // 8)
    w13, s13 = mla_moe.quantize_rows_int8(torch.randn(e, 2 * inter, cols, generator=g))
    w2, s2 = mla_moe.quantize_rows_int8(torch.randn(e, cols, inter, generator=g))
    idx, wts = torch.tensor([[0, 1]], dtype=torch.int32), torch.ones(1, k)
    sec = _best(lambda: mla_moe.cpu_moe_int8(x, idx, wts, w13, s13, w2, s2, 0.0, threads), repeat)
    touched = k * (2 * inter * cols + cols * inter)
    out.append({"kernel": "int8_w8a8_moe_decode", "ms": sec * 1e3, "weight_gbs": touched / sec / 1e9, "threads": threads})
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="cpu_dot_bench")
    ap.add_argument("--rows", type=int, default=4096)
    ap.add_argument("--cols", type=int, default=4096)
    ap.add_argument("--threads", type=int, default=0)
    ap.add_argument("--repeat", type=int, default=5)
    a = ap.parse_args(argv)
    for r in run(a.rows, a.cols, a.threads, a.repeat):
        print(json.dumps(r))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
