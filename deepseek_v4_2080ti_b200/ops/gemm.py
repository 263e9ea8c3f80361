"""Weight-decoding tcgen05 GEMM front-end (csrc/kernels/gemm_wdec.cu).

``y[T, N] = x[T, K] @ W[N, K]^T`` with bf16 activations and either bf16 weights or FP8 E4M3
weights carrying one scale per 128x128 block; FP8 weights are decoded inside the kernel.
Covers the reference's FP8 block-128 projections (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:988-1199)
and bf16 matvec/matmul (cpp_engine/backends/cuda/kernels/bf16_ops.cu:30-167).
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib

WF_BF16 = 0
WF_FP8_B128 = 1
NUM_SMS = 148


def prepack_fp8(w: torch.Tensor) -> torch.Tensor:
    """FP8 weight [N, K] -> the kernel's tile-major layout [ceil(N/128), ceil(K/64), 128, 64] (uint8).

    Two transformations, both done once at load time:
    * every 4 consecutive bytes (w0,w1,w2,w3) are stored as (w0,w2,w1,w3): the decode warps turn one
      32-bit word into two bf16x2 words with shifts and masks only, and this order makes those words
      come out as (w0,w1) and (w2,w3);
    * each [128 rows x 64 bytes] pipeline-stage tile is contiguous (8 KB), so a stage is fetched with a
      single bulk copy instead of 128 separate 64-byte rows.
    """
    u = w.view(torch.uint8)
    n, k = u.shape
    npad, kpad = (n + 127) // 128 * 128, (k + 63) // 64 * 64
    if (npad, kpad) != (n, k):
        full = torch.zeros(npad, kpad, dtype=torch.uint8, device=u.device)
        full[:n, :k] = u
        u = full
    u = u.view(npad, kpad // 4, 4)[:, :, [0, 2, 1, 3]].reshape(npad // 128, 128, kpad // 64, 64)
    return u.permute(0, 2, 1, 3).contiguous()


@dataclass
class PackedLinear:
    """A weight matrix as the GEMM kernel consumes it."""
    wfmt: int
    weight: torch.Tensor          # uint8 [N, K] (prepacked fp8) or bf16 [N, K]
    scales: torch.Tensor | None   # fp32 [ceil(N/128), ceil(K/128)]
    n: int
    k: int

    @staticmethod
    def from_fp8(w_fp8: torch.Tensor, scale: torch.Tensor) -> "PackedLinear":
        n, k = w_fp8.shape
        return PackedLinear(WF_FP8_B128, prepack_fp8(w_fp8), scale.float().contiguous(), n, k)

    @staticmethod
    def from_bf16(w: torch.Tensor) -> "PackedLinear":
        n, k = w.shape
        return PackedLinear(WF_BF16, w.to(torch.bfloat16).contiguous(), None, n, k)

    def nbytes(self) -> int:
        return self.weight.numel() * self.weight.element_size() + (0 if self.scales is None else self.scales.numel() * 4)


_workspaces: dict[tuple[int, int], torch.Tensor] = {}


def _workspace(nfloats: int, device) -> torch.Tensor:
    key = (torch.device(device).index or 0, 0)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nfloats:
        ws = torch.empty(max(nfloats, 1 << 22), dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def pick_splits(t: int, n: int, k: int) -> int:
    """Split K when the tile grid alone cannot fill the 148 SMs (small-batch decode)."""
    bn = 16 if t <= 16 else 32 if t <= 32 else 64 if t <= 64 else 128 if t <= 128 else 256
    tiles = ((n + 127) // 128) * ((t + bn - 1) // bn)
    if tiles >= NUM_SMS or t > 128:
        return 1
    kb = (k + 63) // 64
    s = max(1, min(NUM_SMS // tiles, kb // 8))
    return s


def linear(x: torch.Tensor, w: PackedLinear, residual: torch.Tensor | None = None,
           out: torch.Tensor | None = None, splits: int | None = None,
           out_f32: bool = False) -> torch.Tensor:
    """``x [T, K] bf16`` -> ``[T, N]`` bf16 (or fp32 when ``out_f32``)."""
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.dim() == 2 and x.is_contiguous()
    t, k = x.shape
    assert k == w.k, (k, w.k)
    n = w.n
    if splits is None:
        splits = 1 if out_f32 else pick_splits(t, n, k)
    L = _lib.lib()
    st = _lib.status_word(x.device)
    if out_f32:
        o32 = out if out is not None else torch.empty(t, n, dtype=torch.float32, device=x.device)
        rc = L.b200_gemm_wdec(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x), None,
                              _lib.ptr(o32), None, t, n, k, 1, _lib.ptr(st), _lib.stream())
        _lib.check(rc, "gemm_wdec")
        return o32
    if out is None:
        out = torch.empty(t, n, dtype=torch.bfloat16, device=x.device)
    if splits <= 1:
        rc = L.b200_gemm_wdec(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x), _lib.ptr(out),
                              None, _lib.ptr(residual), t, n, k, 1, _lib.ptr(st), _lib.stream())
        _lib.check(rc, "gemm_wdec")
        return out
    kb = (k + 63) // 64
    splits = min(splits, kb)
    per = (kb + splits - 1) // splits
    splits = (kb + per - 1) // per          # same rule as the launcher: no empty split
    ws = _workspace(splits * t * n, x.device)
    rc = L.b200_gemm_wdec(w.wfmt, _lib.ptr(w.weight), _lib.ptr(w.scales), _lib.ptr(x), None, _lib.ptr(ws),
                          None, t, n, k, splits, _lib.ptr(st), _lib.stream())
    _lib.check(rc, "gemm_wdec(split-k)")
    rc = L.b200_splitk_reduce(_lib.ptr(ws), splits, ctypes.c_longlong(t * n), _lib.ptr(residual),
                              _lib.ptr(out), _lib.stream())
    _lib.check(rc, "splitk_reduce")
    return out


def linear_ref(x: torch.Tensor, w_fp32: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 oracle: x @ w^T (+ residual)."""
    y = x.float() @ w_fp32.float().t()
    if residual is not None:
        y = y + residual.float()
    return y
