"""GGUF-quantised linear layers on the tensor cores (csrc/kernels/gemm_wdec_gguf.cu).

The raw GGUF blocks are only *regrouped* at load time so that every pipeline stage of the GEMM (128 output rows x 64
inputs) is one contiguous block ``[128 x quant bytes | 128 x scale bytes]``; the quantised codes stay as they are and
are decoded in registers inside the kernel.  Supported: Q8_0, Q4_K, Q5_K, Q6_K, Q3_K, Q2_K, IQ1_M, IQ2_XXS, IQ2_XS,
IQ3_XXS, IQ4_XS."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ..formats.gguf import GGMLType
from ..formats.gguf.quant import _unpack_scale_min_6bit, tables
from . import _lib

WF = {GGMLType.Q8_0: 3, GGMLType.Q4_K: 4, GGMLType.Q2_K: 5, GGMLType.IQ2_XXS: 6, GGMLType.Q5_K: 7, GGMLType.IQ3_XXS: 8,
      GGMLType.IQ1_M: 9, GGMLType.Q6_K: 10, GGMLType.Q3_K: 11, GGMLType.IQ4_XS: 12, GGMLType.IQ2_XS: 13}
_LUT_TYPES = (GGMLType.IQ2_XXS, GGMLType.IQ3_XXS, GGMLType.IQ1_M, GGMLType.IQ4_XS, GGMLType.IQ2_XS)
_lut: dict[tuple, torch.Tensor] = {}


def codebook(device) -> torch.Tensor:
    """IQ2_XXS codebook (256 x 8 magnitudes) followed by the 128-entry sign table, as bytes on ``device``."""
    return lut_for(GGMLType.IQ2_XXS, device)


def lut_for(t, device) -> torch.Tensor | None:
    """Codebook table a format's in-register decode reads (None when it needs none): IQ2_XXS 256 x 8 magnitudes +
    128 sign bytes; IQ3_XXS 256 x 4 magnitudes + 128 sign bytes; IQ1_M 2048 x 8 int8 grid values; IQ4_XS the 16 int8
    code values; IQ2_XS 512 x 8 magnitudes + 128 sign bytes."""
    t = GGMLType(t)
    if t not in _LUT_TYPES:
        return None
    key = (t, torch.device(device).index or 0)
    if key not in _lut:
        tb = tables("cpu")
        if t == GGMLType.IQ2_XXS:
            v = torch.cat([tb["iq2xxs"].to(torch.uint8).reshape(-1), tb["ksigns"]])
        elif t == GGMLType.IQ3_XXS:
            v = torch.cat([tb["iq3xxs"].to(torch.uint8).reshape(-1), tb["ksigns"]])
        elif t == GGMLType.IQ4_XS:
            v = tb["iq4nl"].to(torch.int8).reshape(-1).view(torch.uint8)
        elif t == GGMLType.IQ2_XS:
            v = torch.cat([tb["iq2xs"].to(torch.uint8).reshape(-1), tb["ksigns"]])
        else:
            v = tb["iq1"].to(torch.int8).reshape(-1).view(torch.uint8)
        _lut[key] = v.contiguous().to(device)
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
    if t == GGMLType.Q5_K:
        b = raw.view(n, nb, 176)
        sc, mn = _unpack_scale_min_6bit(b[:, :, 4:16].reshape(-1, 12))
        sc, mn = sc.view(n, nb, 4, 2), mn.view(n, nb, 4, 2)
        qs = b[:, :, 48:176].reshape(n, nb, 4, 32)
        qh = b[:, :, 16:48].to(torch.int64)                                 # [n, nb, 32]: bit j = fifth bit of sub-block j
        pw = (1 << torch.arange(32, device=raw.device, dtype=torch.int64))
        masks = torch.stack([(((qh >> j) & 1) * pw).sum(-1) for j in range(8)], -1)      # [n, nb, 8] 32-bit masks
        mb = torch.stack([(masks >> (8 * i)) & 0xFF for i in range(4)], -1).to(torch.uint8)   # [n, nb, 8, 4] little-endian
        q = torch.cat([qs, mb.view(n, nb, 4, 8)], -1).reshape(n, nb * 4, 40)
        dd = b[:, :, None, 0:4].expand(n, nb, 4, 4)
        s = torch.cat([dd, torch.stack([sc[..., 0], mn[..., 0], sc[..., 1], mn[..., 1]], -1).to(torch.uint8)], -1)
        return _tile(q, s.reshape(n, nb * 4, 8))
    if t == GGMLType.IQ3_XXS:
        b = raw.view(n, nb, 98)
        q = torch.cat([b[:, :, 2:66].reshape(n, nb, 4, 16), b[:, :, 66:98].reshape(n, nb, 4, 8)], -1).reshape(n, nb * 4, 24)
        s = torch.cat([b[:, :, None, 0:2].expand(n, nb, 4, 2), b.new_zeros(n, nb, 4, 2)], -1).reshape(n, nb * 4, 4)
        return _tile(q, s)
    if t == GGMLType.IQ1_M:
        b = raw.view(n, nb, 56)
        sc = b[:, :, 48:56].to(torch.int32)
        sc16 = sc[:, :, 0::2] | (sc[:, :, 1::2] << 8)                       # [n, nb, 4]
        dbits = sum(((sc16[:, :, i] >> 12) & 0xF) << (4 * i) for i in range(4))
        dby = torch.stack([dbits & 0xFF, dbits >> 8], -1).to(torch.uint8)   # fp16 d, little-endian
        s3 = torch.stack([(sc16 >> (3 * i)) & 7 for i in range(4)], -1).reshape(n, nb, 16)
        pair = (s3[:, :, 0::2] | (s3[:, :, 1::2] << 3)).to(torch.uint8).view(n, nb, 4, 2)   # one byte per 32 inputs
        q = torch.cat([b[:, :, 0:32].reshape(n, nb, 4, 8), b[:, :, 32:48].reshape(n, nb, 4, 4)], -1).reshape(n, nb * 4, 12)
        s = torch.cat([dby[:, :, None, :].expand(n, nb, 4, 2), pair], -1).reshape(n, nb * 4, 4)
        return _tile(q.contiguous(), s.contiguous())
    if t == GGMLType.Q6_K:
        b = raw.view(n, nb, 210)
        ql = b[:, :, 0:128].view(n, nb, 2, 2, 32)                           # [half, which 32 bytes, l]
        lo = torch.stack([ql & 0xF, ql >> 4], 3)                            # [n, nb, half, p, which, l]: stage = 2 half + p
        nib = (lo[..., 0, :] | (lo[..., 1, :] << 4)).reshape(n, nb * 4, 32)
        qh = b[:, :, 128:192].view(n, nb, 2, 1, 32).to(torch.int64)
        sh = torch.arange(4, device=raw.device).view(1, 1, 1, 4, 1) * 2
        hi = ((qh >> sh) & 3).reshape(n, nb * 4, 2, 32)                     # [stage, half of stage, l] (g = 2 p + hh)
        hw = (hi << (2 * torch.arange(32, device=raw.device))).sum(-1)      # 64-bit word per (stage, hh)
        hb = torch.stack([(hw >> (8 * i)) & 0xFF for i in range(8)], -1).to(torch.uint8).reshape(n, nb * 4, 16)
        q = torch.cat([nib, hb], -1)
        dd = torch.cat([b[:, :, 208:210], b.new_zeros(n, nb, 2)], -1)[:, :, None, :].expand(n, nb, 4, 4)
        s = torch.cat([dd, b[:, :, 192:208].view(n, nb, 4, 4)], -1).reshape(n, nb * 4, 8)
        return _tile(q.contiguous(), s.contiguous())
    if t == GGMLType.Q3_K:
        b = raw.view(n, nb, 110)
        qs = b[:, :, 32:96].view(n, nb, 2, 1, 32).to(torch.int64)
        sh = torch.arange(4, device=raw.device).view(1, 1, 1, 4, 1) * 2
        lo = ((qs >> sh) & 3).reshape(n, nb * 4, 2, 32)                     # element 128 half + 32 s + l -> stage 2 half + s / 2
        lw = (lo << (2 * torch.arange(32, device=raw.device))).sum(-1)
        lb = torch.stack([(lw >> (8 * i)) & 0xFF for i in range(8)], -1).to(torch.uint8).reshape(n, nb * 4, 16)
        hm = b[:, :, 0:32].to(torch.int64)                                  # bit j of byte l = third bit of element 32 j + l
        masks = torch.stack([(((hm >> j) & 1) << torch.arange(32, device=raw.device)).sum(-1) for j in range(8)], -1)
        mb = torch.stack([(masks >> (8 * i)) & 0xFF for i in range(4)], -1).to(torch.uint8).reshape(n, nb * 4, 8)
        q = torch.cat([lb, mb], -1)
        sc = b[:, :, 96:108].to(torch.int64)
        lsc = torch.stack([sc[..., :8] & 0xF, sc[..., :8] >> 4], 2).reshape(n, nb, 16)
        hsc = torch.stack([(sc[..., 8:12] >> (2 * j)) & 3 for j in range(4)], 2).reshape(n, nb, 16)
        s6 = ((lsc | (hsc << 4)) - 32).to(torch.int8).view(torch.uint8).view(n, nb, 4, 4)
        dd = torch.cat([b[:, :, 108:110], b.new_zeros(n, nb, 2)], -1)[:, :, None, :].expand(n, nb, 4, 4)
        s = torch.cat([dd, s6], -1).reshape(n, nb * 4, 8)
        return _tile(q.contiguous(), s.contiguous())
    if t == GGMLType.IQ4_XS:
        b = raw.view(n, nb, 136)
        sh = b[:, :, 2].to(torch.int64) | (b[:, :, 3].to(torch.int64) << 8)
        slb = b[:, :, 4:8].to(torch.int64)
        sl = torch.stack([slb & 0xF, slb >> 4], -1).reshape(n, nb, 8)
        s6 = (sl | (torch.stack([(sh >> (2 * i)) & 3 for i in range(8)], -1) << 4)) - 32
        q = b[:, :, 8:136].reshape(n, nb * 4, 32)
        s = torch.cat([b[:, :, None, 0:2].expand(n, nb, 4, 2), s6.to(torch.int8).view(torch.uint8).view(n, nb, 4, 2)], -1)
        return _tile(q, s.reshape(n, nb * 4, 4).contiguous())
    if t == GGMLType.IQ2_XS:
        b = raw.view(n, nb, 74)
        q = b[:, :, 2:66].reshape(n, nb * 4, 16)
        s = torch.cat([b[:, :, None, 0:2].expand(n, nb, 4, 2), b[:, :, 66:74].view(n, nb, 4, 2)], -1).reshape(n, nb * 4, 4)
        return _tile(q, s.contiguous())
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
    lut = lut_for(w.ggml_type, x.device)
    if not out_f32 and t <= 128:
        from . import gemm
        splits = gemm.pick_splits(t, w.n, w.k)
        if splits > 1:
            ws, counters = gemm._workspace(splits * t * w.n, x.device)
            rc = _lib.lib().b200_gemm_wdec_gguf_splitk(WF[w.ggml_type], _lib.ptr(w.weight), _lib.ptr(lut), _lib.ptr(x),
                                                       _lib.ptr(out), _lib.ptr(ws), _lib.ptr(residual), t, w.n, w.k, splits,
                                                       _lib.ptr(counters), _lib.ptr(_lib.status_word(x.device)), _lib.stream())
            _lib.check(rc, "gemm_wdec_gguf(split-k)")
            return out
    rc = _lib.lib().b200_gemm_wdec_gguf(WF[w.ggml_type], _lib.ptr(w.weight), _lib.ptr(lut), _lib.ptr(x),
                                        None if out_f32 else _lib.ptr(out), _lib.ptr(out) if out_f32 else None,
                                        _lib.ptr(residual), t, w.n, w.k, _lib.ptr(_lib.status_word(x.device)), _lib.stream())
    _lib.check(rc, "gemm_wdec_gguf")
    return out
