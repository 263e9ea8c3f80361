"""GGUF-quantised linear layers on the tensor cores (csrc/kernels/gemm_wdec_gguf.cu).

The raw GGUF blocks are only *regrouped* at load time so that every pipeline stage of the GEMM (128 output rows x 64
inputs) is one contiguous block ``[128 x quant bytes | 128 x scale bytes]``; the quantised codes stay as they are and
are decoded in registers inside the kernel.  Supported: Q8_0, Q4_K, Q2_K, IQ2_XXS."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ..formats.gguf import GGMLType
from ..formats.gguf.quant import _unpack_scale_min_6bit, tables
from . import _lib

WF = {GGMLType.Q8_0: 3, GGMLType.Q4_K: 4, GGMLType.Q2_K: 5, GGMLType.IQ2_XXS: 6}
_lut: dict[int, torch.Tensor] = {}


def codebook(device) -> torch.Tensor:
    """IQ2_XXS codebook (256 x 8 magnitudes) followed by the 128-entry sign table, as bytes on ``device``."""
    key = torch.device(device).index or 0
    if key not in _lut:
        t = tables("cpu")
        _lut[key] = torch.cat([t["iq2xxs"].to(torch.uint8).reshape(-1), t["ksigns"]]).to(device)
    return _lut[key]


def _tile(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    """q [N, KB, QB], s [N, KB, SB] -> [ceil(N/128), KB, 128*QB + 128*SB] (rows zero-padded to a multiple of 128)."""
    n, kb, qb = q.shape
    sb = s.shape[2]
    npad = (n + 127) // 128 * 128
    if npad != n:
        q = torch.cat([q, q.new_zeros(npad - n, kb, qb)])
        s = torch.cat([s, s.new_zeros(npad - n, kb, sb)])
    qt = q.view(npad // 128, 128, kb, qb).permute(0, 2, 1, 3).reshape(npad // 128, kb, 128 * qb)
    st = s.view(npad // 128, 128, kb, sb).permute(0, 2, 1, 3).reshape(npad // 128, kb, 128 * sb)
    return torch.cat([qt, st], -1).contiguous()


def prepack(raw: torch.Tensor, t: GGMLType, k: int) -> torch.Tensor:
    """Raw GGUF blocks ``uint8 [N, row_bytes]`` -> the kernel's stage-major layout (uint8)."""
    t = GGMLType(t)
    n = raw.shape[0]
    assert k % 64 == 0
    if t == GGMLType.Q8_0:
        b = raw.view(n, k // 32, 34)
        q = b[:, :, 2:].reshape(n, k // 64, 64)
        s = b[:, :, :2].reshape(n, k // 64, 4)
        return _tile(q, s)
    assert k % 256 == 0
    nb = k // 256
    if t == GGMLType.Q4_K:
        b = raw.view(n, nb, 144)
        sc, mn = _unpack_scale_min_6bit(b[:, :, 4:16].reshape(-1, 12))
        sc, mn = sc.view(n, nb, 4, 2), mn.view(n, nb, 4, 2)
        q = b[:, :, 16:].reshape(n, nb * 4, 32)
        dd = b[:, :, None, 0:4].expand(n, nb, 4, 4)
        s = torch.cat([dd, torch.stack([sc[..., 0], mn[..., 0], sc[..., 1], mn[..., 1]], -1).to(torch.uint8)], -1)
        return _tile(q, s.reshape(n, nb * 4, 8))
    if t == GGMLType.Q2_K:
        b = raw.view(n, nb, 84)
        qs = b[:, :, 16:80].view(n, nb, 2, 1, 32)                        # [half, -, byte]
        shifts = torch.tensor([0, 4], dtype=torch.uint8, device=raw.device).view(1, 1, 1, 2, 1)
        nib = (qs >> shifts) & 0xF                                       # [n, nb, half, stage-in-half, 32]
        nib = nib.reshape(n, nb * 4, 32)
        q = nib[:, :, :16] | (nib[:, :, 16:] << 4)
        dd = b[:, :, None, 80:84].expand(n, nb, 4, 4)
        s = torch.cat([dd, b[:, :, 0:16].view(n, nb, 4, 4)], -1).reshape(n, nb * 4, 8)
        return _tile(q.contiguous(), s)
    if t == GGMLType.IQ2_XXS:
        b = raw.view(n, nb, 66)
        q = b[:, :, 2:].reshape(n, nb * 4, 16)
        s = torch.cat([b[:, :, None, 0:2].expand(n, nb, 4, 2), b.new_zeros(n, nb, 4, 2)], -1).reshape(n, nb * 4, 4)
        return _tile(q, s)
    raise ValueError(f"{t.name} has no tensor-core decode path yet")


@dataclass
class GGUFLinear:
    ggml_type: GGMLType
    weight: torch.Tensor          # packed stages
    n: int
    k: int

    @staticmethod
    def from_raw(raw: torch.Tensor, t: GGMLType, n: int, k: int, device="cuda") -> "GGUFLinear":
        return GGUFLinear(GGMLType(t), prepack(raw.to(device), t, k), n, k)

    def nbytes(self) -> int:
        return self.weight.numel()


def linear(x: torch.Tensor, w: GGUFLinear, residual: torch.Tensor | None = None, out_f32: bool = False) -> torch.Tensor:
    """``x [T, K] bf16`` -> ``[T, N]``: the GGUF blocks are decoded inside the GEMM."""
    assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[1] == w.k
    t = x.shape[0]
    out = torch.empty(t, w.n, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    lut = codebook(x.device) if w.ggml_type == GGMLType.IQ2_XXS else None
    rc = _lib.lib().b200_gemm_wdec_gguf(WF[w.ggml_type], _lib.ptr(w.weight), _lib.ptr(lut), _lib.ptr(x),
                                        None if out_f32 else _lib.ptr(out), _lib.ptr(out) if out_f32 else None,
                                        _lib.ptr(residual), t, w.n, w.k, _lib.ptr(_lib.status_word(x.device)), _lib.stream())
    _lib.check(rc, "gemm_wdec_gguf")
    return out
