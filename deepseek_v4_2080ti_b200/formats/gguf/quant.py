"""Block quantisers and reference dequantisers for the GGUF types this engine serves, written with torch ops so
they run on the CPU (tests) and on the GPU (synthesising large checkpoints).

Every function works on a 2-D weight ``[rows, cols]`` <-> raw block bytes ``uint8 [rows, cols / block * block_bytes]``.
Layouts follow ggml (the ``gguf`` Python package is the independent oracle in the tests); the IQ codebooks
(2-bit 256 x 8, 3-bit 256 x 4, 1-bit 2048 x 8, and the 128-entry sign table) are format constants and are taken
from that package at first use rather than being duplicated here.

The i-quant quantisers are plain nearest-codeword searches (no importance matrix): good enough to synthesise
checkpoints whose blocks are valid and whose values track the source tensor.
"""
from __future__ import annotations

import numpy as np
import torch

from .constants import BLOCK_BYTES, BLOCK_ELEMS, QK_K, GGMLType

_tables: dict[str, torch.Tensor] = {}


def tables(device="cpu") -> dict[str, torch.Tensor]:
    """Codebooks as float32 tensors: iq2xxs [256, 8], iq2xs [512, 8], iq3xxs [256, 4], iq1 [2048, 8], iq4nl [16];
    ksigns uint8 [128]."""
    if not _tables:
        try:
            from gguf import quants as gq
        except Exception as exc:  # pragma: no cover - image always has it
            raise RuntimeError("the IQ codebooks are read from the 'gguf' Python package, which is not importable") from exc
        for cls in (gq.IQ2_XXS, gq.IQ2_XS, gq.IQ3_XXS, gq.IQ1_M):
            cls.init_grid()
        _tables["iq2xs"] = torch.from_numpy(np.ascontiguousarray(gq.IQ2_XS.grid.reshape(512, 8))).float()
        _tables["iq4nl"] = torch.tensor(list(gq.IQ4_NL.kvalues), dtype=torch.float32)
        _tables["iq2xxs"] = torch.from_numpy(np.ascontiguousarray(gq.IQ2_XXS.grid.reshape(256, 8))).float()
        _tables["iq3xxs"] = torch.from_numpy(np.ascontiguousarray(gq.IQ3_XXS.grid.reshape(256, 4))).float()
        _tables["iq1"] = torch.from_numpy(np.ascontiguousarray(gq.IQ1_M.grid.reshape(2048, 8))).float()
        _tables["ksigns"] = torch.from_numpy(np.frombuffer(gq.IQ2_XXS.ksigns, dtype=np.uint8).copy())
        _tables["iq1_delta"] = torch.tensor(float(gq.IQ1_M.delta))
    return {k: v.to(device) for k, v in _tables.items()}


def _f16_bytes(x: torch.Tensor) -> torch.Tensor:
    """float tensor [...] -> uint8 [..., 2] (little-endian fp16)."""
    return x.to(torch.float16).contiguous().view(torch.uint8).reshape(*x.shape, 2)


def _bytes_f16(b: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 2] -> float32 [...]."""
    return b.contiguous().view(torch.float16).reshape(b.shape[:-1]).float()


def _blocks(w: torch.Tensor, n: int) -> torch.Tensor:
    rows, cols = w.shape
    assert cols % n == 0, (cols, n)
    return w.float().reshape(rows * cols // n, n)


# ----------------------------------------------------------------------------- Q8_0
def _q_q8_0(w):
    b = _blocks(w, 32)
    d = b.abs().amax(1, keepdim=True) / 127.0
    q = torch.where(d > 0, b / d.clamp_min(1e-30), torch.zeros_like(b)).round().clamp(-127, 127).to(torch.int8)
    return torch.cat([_f16_bytes(d[:, 0]), q.view(torch.uint8)], 1)


def _d_q8_0(b):
    return _bytes_f16(b[:, :2])[:, None] * b[:, 2:].contiguous().view(torch.int8).float()


# ----------------------------------------------------------------------------- k-quant helpers
def _pack_scale_min_6bit(sc: torch.Tensor, mn: torch.Tensor) -> torch.Tensor:
    """sc, mn: uint8 [n, 8] (6-bit values) -> 12 bytes in the Q4_K / Q5_K packing."""
    sc, mn = sc.to(torch.uint8), mn.to(torch.uint8)
    out = torch.zeros(sc.shape[0], 12, dtype=torch.uint8, device=sc.device)
    out[:, 0:4] = (sc[:, 0:4] & 0x3F) | ((sc[:, 4:8] >> 4) << 6)
    out[:, 4:8] = (mn[:, 0:4] & 0x3F) | ((mn[:, 4:8] >> 4) << 6)
    out[:, 8:12] = (sc[:, 4:8] & 0x0F) | ((mn[:, 4:8] & 0x0F) << 4)
    return out


def _unpack_scale_min_6bit(s: torch.Tensor):
    d, m, md = s[:, 0:4], s[:, 4:8], s[:, 8:12]
    sc = torch.cat([d & 0x3F, (md & 0x0F) | ((d >> 2) & 0x30)], 1)
    mn = torch.cat([m & 0x3F, (md >> 4) | ((m >> 2) & 0x30)], 1)
    return sc, mn


def _affine_subblocks(b: torch.Tensor, sub: int, qmax: int, smax: int):
    """Per sub-block affine quantisation x ~= d*sc*q - dmin*mn*1 with q in [0, qmax], sc/mn in [0, smax]:
    returns (d, dmin [n], sc, mn [n, nsub] uint8, q [n, 256] uint8)."""
    n = b.shape[0]
    x = b.view(n, QK_K // sub, sub)
    lo = x.amin(-1).clamp_max(0.0)
    hi = x.amax(-1)
    scale = ((hi - lo) / qmax).clamp_min(1e-12)          # per sub-block step
    mins = -lo                                           # >= 0
    d = (scale.amax(-1) / smax).clamp_min(1e-12)
    dmin = (mins.amax(-1) / smax).clamp_min(1e-12)
    d = d.to(torch.float16).float().clamp_min(6e-8)      # what the block stores
    dmin = dmin.to(torch.float16).float().clamp_min(6e-8)
    sc = (scale / d[:, None]).round().clamp(0, smax)
    mn = (mins / dmin[:, None]).round().clamp(0, smax)
    eff_s = (d[:, None] * sc).clamp_min(1e-12)
    q = ((x + (dmin[:, None] * mn)[..., None]) / eff_s[..., None]).round().clamp(0, qmax)
    q = torch.where((sc > 0)[..., None], q, torch.zeros_like(q))
    return d, dmin, sc.to(torch.uint8), mn.to(torch.uint8), q.to(torch.uint8).view(n, QK_K)


# ----------------------------------------------------------------------------- Q4_K / Q5_K
def _q_q4_k(w):
    b = _blocks(w, QK_K)
    d, dmin, sc, mn, q = _affine_subblocks(b, 32, 15, 63)
    q = q.view(-1, 4, 2, 32)                              # 64-element groups: low nibbles = first 32, high = next 32
    qs = (q[:, :, 0] | (q[:, :, 1] << 4)).reshape(-1, 128)
    return torch.cat([_f16_bytes(d), _f16_bytes(dmin), _pack_scale_min_6bit(sc, mn), qs], 1)


def _d_q4_k(b):
    d, dmin = _bytes_f16(b[:, 0:2]), _bytes_f16(b[:, 2:4])
    sc, mn = _unpack_scale_min_6bit(b[:, 4:16])
    qs = b[:, 16:144].view(-1, 4, 1, 32)
    q = torch.cat([qs & 0x0F, qs >> 4], 2).reshape(-1, 8, 32).float()
    return ((d[:, None] * sc.float())[..., None] * q - (dmin[:, None] * mn.float())[..., None]).reshape(-1, QK_K)


def _q_q5_k(w):
    b = _blocks(w, QK_K)
    d, dmin, sc, mn, q = _affine_subblocks(b, 32, 31, 63)
    q = q.view(-1, 8, 32)
    ql = (q & 0x0F).view(-1, 4, 2, 32)
    qs = (ql[:, :, 0] | (ql[:, :, 1] << 4)).reshape(-1, 128)
    hb = (q >> 4) & 1                                    # [n, 8, 32]: bit j of qh[l] is the high bit of sub-block j
    shifts = torch.arange(8, device=w.device, dtype=torch.uint8).view(1, 8, 1)
    qh = (hb << shifts).sum(1).to(torch.uint8)
    return torch.cat([_f16_bytes(d), _f16_bytes(dmin), _pack_scale_min_6bit(sc, mn), qh, qs], 1)


def _d_q5_k(b):
    d, dmin = _bytes_f16(b[:, 0:2]), _bytes_f16(b[:, 2:4])
    sc, mn = _unpack_scale_min_6bit(b[:, 4:16])
    qh = b[:, 16:48]
    qs = b[:, 48:176].view(-1, 4, 1, 32)
    ql = torch.cat([qs & 0x0F, qs >> 4], 2).reshape(-1, 8, 32)
    shifts = torch.arange(8, device=b.device, dtype=torch.uint8).view(1, 8, 1)
    hb = (qh[:, None, :] >> shifts) & 1
    q = (ql | (hb << 4)).float()
    return ((d[:, None] * sc.float())[..., None] * q - (dmin[:, None] * mn.float())[..., None]).reshape(-1, QK_K)


# ----------------------------------------------------------------------------- Q2_K
def _q_q2_k(w):
    b = _blocks(w, QK_K)
    d, dmin, sc, mn, q = _affine_subblocks(b, 16, 3, 15)
    scales = (sc & 0x0F) | (mn << 4)                      # [n, 16]
    q = q.view(-1, 2, 4, 32)                              # 128-element halves; 4 two-bit planes of 32
    shifts = torch.tensor([0, 2, 4, 6], device=w.device, dtype=torch.uint8).view(1, 1, 4, 1)
    qs = (q << shifts).sum(2).to(torch.uint8).reshape(-1, 64)
    return torch.cat([scales, qs, _f16_bytes(d), _f16_bytes(dmin)], 1)


def _d_q2_k(b):
    scales, qs = b[:, 0:16], b[:, 16:80]
    d, dmin = _bytes_f16(b[:, 80:82]), _bytes_f16(b[:, 82:84])
    dl = d[:, None] * (scales & 0x0F).float()
    ml = dmin[:, None] * (scales >> 4).float()
    shifts = torch.tensor([0, 2, 4, 6], device=b.device, dtype=torch.uint8).view(1, 1, 4, 1)
    q = ((qs.view(-1, 2, 1, 32) >> shifts) & 3).reshape(-1, 16, 16).float()
    return (dl[..., None] * q - ml[..., None]).reshape(-1, QK_K)


# ----------------------------------------------------------------------------- sign packing shared by IQ2_XXS / IQ3_XXS
def _sign_index(neg: torch.Tensor, mag: torch.Tensor):
    """neg: bool [..., 8]; mag: float [..., 8].  The format stores 7 sign bits; the 8th makes the parity even.
    Where the parity is odd the sign of the smallest-magnitude element is flipped.  Returns (7-bit index, neg)."""
    odd = (neg.sum(-1) % 2) == 1
    flip = torch.zeros_like(neg)
    flip.scatter_(-1, mag.argmin(-1, keepdim=True), True)
    neg = torch.where(odd[..., None] & flip, ~neg, neg)
    bits = (neg[..., :7].long() << torch.arange(7, device=neg.device)).sum(-1)
    return bits, neg


def _signs_from_index(idx: torch.Tensor, ksigns: torch.Tensor) -> torch.Tensor:
    s = ksigns[idx.long()]
    bits = (s[..., None] >> torch.arange(8, device=idx.device, dtype=torch.uint8)) & 1
    return 1.0 - 2.0 * bits.float()


def _nearest(mag: torch.Tensor, grid: torch.Tensor, chunk: int = 1 << 16) -> torch.Tensor:
    """mag [n, k] -> index of the nearest row of grid [g, k] (squared distance), in chunks to bound memory."""
    out = torch.empty(mag.shape[0], dtype=torch.long, device=mag.device)
    g2 = (grid * grid).sum(1)
    for s in range(0, mag.shape[0], chunk):
        m = mag[s:s + chunk]
        out[s:s + chunk] = (g2[None, :] - 2.0 * m @ grid.t()).argmin(1)
    return out


# ----------------------------------------------------------------------------- IQ2_XXS
def _q_iq2_xxs(w):
    t = tables(w.device)
    b = _blocks(w, QK_K)
    n = b.shape[0]
    x = b.view(n, 8, 4, 8)                                # 8 groups of 32 = 4 x 8
    amax = x.abs().amax((1, 2, 3)).clamp_min(1e-12)
    # value = d * (0.5 + s) * 0.25 * grid * sign, grid up to 43, s in 0..15
    d = (amax / (43.0 * 0.25 * 15.5)).to(torch.float16).float().clamp_min(6e-8)
    gmax = x.abs().amax((2, 3))                           # [n, 8]
    s = (gmax / (d[:, None] * 0.25 * 43.0) - 0.5).round().clamp(0, 15)
    db = d[:, None] * (0.5 + s) * 0.25
    mag = (x.abs() / db[..., None, None]).reshape(-1, 8)
    gi = _nearest(mag, t["iq2xxs"]).view(n, 8, 4)
    sidx, _ = _sign_index((x < 0).reshape(n, 8, 4, 8), x.abs().reshape(n, 8, 4, 8))
    w0 = (gi[..., 0] | (gi[..., 1] << 8) | (gi[..., 2] << 16) | (gi[..., 3] << 24)).to(torch.int64)
    w1 = (sidx[..., 0] | (sidx[..., 1] << 7) | (sidx[..., 2] << 14) | (sidx[..., 3] << 21) | (s.long() << 28)).to(torch.int64)
    words = torch.stack([w0, w1], -1).reshape(n, 16)
    qs = torch.stack([(words >> (8 * i)) & 0xFF for i in range(4)], -1).to(torch.uint8).reshape(n, 64)
    return torch.cat([_f16_bytes(d), qs], 1)


def _u32(b: torch.Tensor) -> torch.Tensor:
    """uint8 [..., 4k] -> int64 [..., k] little-endian words."""
    b = b.reshape(*b.shape[:-1], -1, 4).long()
    return b[..., 0] | (b[..., 1] << 8) | (b[..., 2] << 16) | (b[..., 3] << 24)


def _d_iq2_xxs(b):
    t = tables(b.device)
    n = b.shape[0]
    d = _bytes_f16(b[:, 0:2])
    words = _u32(b[:, 2:66]).view(n, 8, 2)
    w0, w1 = words[..., 0], words[..., 1]
    db = d[:, None] * (0.5 + (w1 >> 28).float()) * 0.25
    gi = torch.stack([(w0 >> (8 * i)) & 0xFF for i in range(4)], -1)
    si = torch.stack([(w1 >> (7 * i)) & 0x7F for i in range(4)], -1)
    return (db[..., None, None] * t["iq2xxs"][gi] * _signs_from_index(si, t["ksigns"])).reshape(n, QK_K)


# ----------------------------------------------------------------------------- IQ3_XXS
def _q_iq3_xxs(w):
    t = tables(w.device)
    b = _blocks(w, QK_K)
    n = b.shape[0]
    x = b.view(n, 8, 4, 8)
    amax = x.abs().amax((1, 2, 3)).clamp_min(1e-12)
    d = (amax / (62.0 * 0.5 * 15.5)).to(torch.float16).float().clamp_min(6e-8)
    gmax = x.abs().amax((2, 3))
    s = (gmax / (d[:, None] * 0.5 * 62.0) - 0.5).round().clamp(0, 15)
    db = d[:, None] * (0.5 + s) * 0.5
    mag = (x.abs() / db[..., None, None]).reshape(-1, 4)          # codewords cover 4 values
    gi = _nearest(mag, t["iq3xxs"]).view(n, 64)
    sidx, _ = _sign_index((x < 0), x.abs())
    w1 = (sidx[..., 0] | (sidx[..., 1] << 7) | (sidx[..., 2] << 14) | (sidx[..., 3] << 21) | (s.long() << 28)).to(torch.int64)
    sc = torch.stack([(w1 >> (8 * i)) & 0xFF for i in range(4)], -1).to(torch.uint8).reshape(n, 32)
    return torch.cat([_f16_bytes(d), gi.to(torch.uint8), sc], 1)


def _d_iq3_xxs(b):
    t = tables(b.device)
    n = b.shape[0]
    d = _bytes_f16(b[:, 0:2])
    gi = b[:, 2:66].long().view(n, 8, 4, 2)
    w1 = _u32(b[:, 66:98])                                         # [n, 8]
    db = d[:, None] * (0.5 + (w1 >> 28).float()) * 0.5
    si = torch.stack([(w1 >> (7 * i)) & 0x7F for i in range(4)], -1)
    grid = t["iq3xxs"][gi].reshape(n, 8, 4, 8)
    return (db[..., None, None] * grid * _signs_from_index(si, t["ksigns"])).reshape(n, QK_K)


# ----------------------------------------------------------------------------- IQ1_M
def _q_iq1_m(w):
    """56 bytes: qs[32] (low 8 bits of 32 codeword indices), qh[16] (3 high bits + delta-sign bit per index),
    scales[8] (sixteen 3-bit scales and the fp16 super-scale spread over the top nibbles of four uint16)."""
    t = tables(w.device)
    b = _blocks(w, QK_K)
    n = b.shape[0]
    x = b.view(n, 16, 2, 8)                               # 16 sub-blocks of 16 = 2 codewords of 8
    delta = float(t["iq1_delta"])
    amax = x.abs().amax((1, 2, 3)).clamp_min(1e-12)
    d = (amax / ((1.0 + delta) * 15.0)).to(torch.float16).float().clamp_min(6e-8)
    smax = x.abs().amax((2, 3))                           # [n, 16]
    s = ((smax / (d[:, None] * (1.0 + delta)) - 1.0) / 2.0).round().clamp(0, 7)
    dl = d[:, None] * (2.0 * s + 1.0)
    y = (x / dl[..., None, None]).reshape(-1, 8)
    grid = t["iq1"]
    ip = _nearest(y - delta, grid)
    im = _nearest(y + delta, grid)
    ep = ((grid[ip] + delta - y) ** 2).sum(1)
    em = ((grid[im] - delta - y) ** 2).sum(1)
    neg = em < ep
    idx = torch.where(neg, im, ip).view(n, 32)
    neg = neg.view(n, 32)
    qs = (idx & 0xFF).to(torch.uint8)
    hi = ((idx >> 8) & 7) | (neg.long() << 3)             # 4 bits per codeword
    qh = (hi[:, 0::2] | (hi[:, 1::2] << 4)).to(torch.uint8)
    s = s.long().view(n, 4, 4)
    sc16 = s[..., 0] | (s[..., 1] << 3) | (s[..., 2] << 6) | (s[..., 3] << 9)
    dbits = d.to(torch.float16).view(torch.int16).long() & 0xFFFF
    sc16 = sc16 | torch.stack([((dbits >> (4 * i)) & 0xF) << 12 for i in range(4)], -1)
    scales = torch.stack([sc16 & 0xFF, sc16 >> 8], -1).to(torch.uint8).reshape(n, 8)
    return torch.cat([qs, qh, scales], 1)


def _d_iq1_m(b):
    t = tables(b.device)
    n = b.shape[0]
    qs, qh, sc = b[:, 0:32].long(), b[:, 32:48].long(), b[:, 48:56].long()
    sc16 = (sc[:, 0::2] | (sc[:, 1::2] << 8))             # [n, 4]
    dbits = sum(((sc16[:, i] >> 12) & 0xF) << (4 * i) for i in range(4))
    d = dbits.to(torch.int16).view(torch.float16).float()
    s = torch.stack([(sc16 >> (3 * i)) & 7 for i in range(4)], -1).reshape(n, 16)
    dl = d[:, None] * (2.0 * s.float() + 1.0)
    hi = torch.stack([qh & 0xF, qh >> 4], -1).reshape(n, 32)
    idx = qs | ((hi & 7) << 8)
    delta = torch.where((hi & 8) == 0, t["iq1_delta"], -t["iq1_delta"])
    vals = t["iq1"][idx] + delta[..., None]               # [n, 32, 8]
    return (dl.repeat_interleave(2, 1)[..., None] * vals).reshape(n, QK_K)


# ----------------------------------------------------------------------------- Q3_K
# block: hmask[32] | qs[64] | scales[12] | d.  16 sub-blocks of 16; value = d * (scale6 - 32) * (q2 - (hbit ? 0 : 4)).
# Element e = 128 h + 32 s + l takes its low bits from (qs[32 h + l] >> 2 s) & 3 and its high bit from bit (4 h + s)
# of hmask[l].
def _q_q3_k(w):
    b = _blocks(w, QK_K)
    n = b.shape[0]
    x = b.view(n, 16, 16)
    amax = x.abs().amax(-1)                                     # [n, 16]
    sub = amax / 4.0                                             # q in [-4, 3]
    d = (sub.amax(-1) / 31.0).to(torch.float16).float().clamp_min(6e-8)
    sc = (sub / d[:, None]).round().clamp(0, 31)                 # stored + 32
    eff = (d[:, None] * sc).clamp_min(1e-12)
    q = (x / eff[..., None]).round().clamp(-4, 3).long() + 4     # 0..7; sub-blocks with scale 0 decode to 0 anyway
    q = q.view(n, 2, 4, 32)                                      # [half, shift, l]
    lo, hi = q & 3, q >> 2
    qs = sum(lo[:, :, s_] << (2 * s_) for s_ in range(4)).to(torch.uint8).reshape(n, 64)
    hm = sum(hi[:, h_, s_] << (4 * h_ + s_) for h_ in range(2) for s_ in range(4)).to(torch.uint8)      # [n, 32]
    s6 = (sc.long() + 32)                                        # 6-bit codes [n, 16]
    lsc = (s6[:, :8] & 0xF) | ((s6[:, 8:] & 0xF) << 4)
    hsc = sum(((s6[:, 4 * j:4 * j + 4] >> 4) & 3) << (2 * j) for j in range(4))
    scales = torch.cat([lsc, hsc], 1).to(torch.uint8)
    return torch.cat([hm, qs, scales, _f16_bytes(d)], 1)


def _d_q3_k(b):
    n = b.shape[0]
    hm, qs, sc, d = b[:, 0:32].long(), b[:, 32:96].long(), b[:, 96:108].long(), _bytes_f16(b[:, 108:110])
    lsc = torch.stack([sc[:, :8] & 0xF, sc[:, :8] >> 4], 1).reshape(n, 16)
    hsc = torch.stack([(sc[:, 8:12] >> (2 * j)) & 3 for j in range(4)], 1).reshape(n, 16)
    s6 = ((lsc | (hsc << 4)) - 32).float()
    ql = torch.stack([(qs.view(n, 2, 32) >> (2 * s_)) & 3 for s_ in range(4)], 2)            # [n, 2, 4, 32]
    qh = torch.stack([(hm >> j) & 1 for j in range(8)], 1).view(n, 2, 4, 32)
    q = (ql - ((qh ^ 1) << 2)).float().reshape(n, 16, 16)
    return ((d[:, None] * s6)[..., None] * q).reshape(n, QK_K)


# ----------------------------------------------------------------------------- Q6_K
# block: ql[128] | qh[64] | scales[16] int8 | d.  value = d * scale * (q6 - 32); element e = 128 h + 32 g + l (g 0..3)
# has low nibble (ql[64 h + 32 (g & 1) + l] >> 4 (g >> 1)) & 15 and high bits (qh[32 h + l] >> 2 g) & 3.
def _q_q6_k(w):
    b = _blocks(w, QK_K)
    n = b.shape[0]
    x = b.view(n, 16, 16)
    sub = x.abs().amax(-1) / 32.0
    d = (sub.amax(-1) / 127.0).to(torch.float16).float().clamp_min(6e-8)
    sc = (sub / d[:, None]).round().clamp(0, 127)
    eff = (d[:, None] * sc).clamp_min(1e-12)
    q = ((x / eff[..., None]).round().clamp(-32, 31).long() + 32).view(n, 2, 4, 32)          # [half, g, l]
    lo, hi = q & 0xF, q >> 4
    ql = torch.stack([lo[:, :, 0] | (lo[:, :, 2] << 4), lo[:, :, 1] | (lo[:, :, 3] << 4)], 2).reshape(n, 128)
    qh = sum(hi[:, :, g_] << (2 * g_) for g_ in range(4)).reshape(n, 64)
    return torch.cat([ql.to(torch.uint8), qh.to(torch.uint8), sc.to(torch.int8).view(torch.uint8), _f16_bytes(d)], 1)


def _d_q6_k(b):
    n = b.shape[0]
    ql, qh = b[:, 0:128].long().view(n, 2, 2, 32), b[:, 128:192].long().view(n, 2, 32)
    sc, d = b[:, 192:208].contiguous().view(torch.int8).float(), _bytes_f16(b[:, 208:210])
    lo = torch.stack([ql[:, :, 0] & 0xF, ql[:, :, 1] & 0xF, ql[:, :, 0] >> 4, ql[:, :, 1] >> 4], 2)      # [n, 2, 4, 32]
    hi = torch.stack([(qh >> (2 * g_)) & 3 for g_ in range(4)], 2)
    q = ((lo | (hi << 4)) - 32).float().reshape(n, 16, 16)
    return ((d[:, None] * sc)[..., None] * q).reshape(n, QK_K)


# ----------------------------------------------------------------------------- IQ2_XS
# block: d | qs[32] uint16 (9-bit index into a 512 x 8 magnitude grid | 7-bit sign index << 9) | scales[8] (two 4-bit
# scales per byte, one per 16 elements).  value = d * (0.5 + s) * 0.25 * grid * sign.
def _q_iq2_xs(w):
    t = tables(w.device)
    b = _blocks(w, QK_K)
    n = b.shape[0]
    x = b.view(n, 16, 2, 8)
    gmaxv = float(t["iq2xs"].max())
    amax = x.abs().amax((1, 2, 3)).clamp_min(1e-12)
    d = (amax / (gmaxv * 0.25 * 15.5)).to(torch.float16).float().clamp_min(6e-8)
    s = (x.abs().amax((2, 3)) / (d[:, None] * 0.25 * gmaxv) - 0.5).round().clamp(0, 15)
    db = d[:, None] * (0.5 + s) * 0.25
    gi = _nearest((x.abs() / db[..., None, None]).reshape(-1, 8), t["iq2xs"]).view(n, 16, 2)
    sidx, _ = _sign_index(x < 0, x.abs())
    q16 = (gi | (sidx << 9)).reshape(n, 32)
    qs = torch.stack([q16 & 0xFF, q16 >> 8], -1).to(torch.uint8).reshape(n, 64)
    sl = s.long().view(n, 8, 2)
    scales = (sl[..., 0] | (sl[..., 1] << 4)).to(torch.uint8)
    return torch.cat([_f16_bytes(d), qs, scales], 1)


def _d_iq2_xs(b):
    t = tables(b.device)
    n = b.shape[0]
    d = _bytes_f16(b[:, 0:2])
    q = b[:, 2:66].long().view(n, 32, 2)
    q16 = q[..., 0] | (q[..., 1] << 8)
    sc = b[:, 66:74].long()
    s = torch.stack([sc & 0xF, sc >> 4], -1).reshape(n, 16).float()
    db = d[:, None] * (0.5 + s) * 0.25
    grid = t["iq2xs"][q16 & 511].view(n, 16, 2, 8)
    signs = _signs_from_index(q16 >> 9, t["ksigns"]).view(n, 16, 2, 8)
    return (db[..., None, None] * grid * signs).reshape(n, QK_K)


# ----------------------------------------------------------------------------- IQ4_XS
# block: d | scales_h uint16 (2 bits per sub-block) | scales_l[4] (4 bits per sub-block) | qs[128].  8 sub-blocks of
# 32: value = d * (scale6 - 32) * kvalues[q4]; sub-block i keeps elements 0..15 in the low nibbles of qs[16 i ..] and
# 16..31 in the high nibbles.
def _q_iq4_xs(w):
    t = tables(w.device)
    kv = t["iq4nl"]
    b = _blocks(w, QK_K)
    n = b.shape[0]
    x = b.view(n, 8, 32)
    # the signed element of largest magnitude maps onto the codebook end of the same sign
    idx = x.abs().argmax(-1, keepdim=True)
    peak = x.gather(-1, idx).squeeze(-1)
    sub = torch.where(peak < 0, peak / kv[0], peak / kv[-1])      # >= 0
    d = (sub.amax(-1) / 31.0).to(torch.float16).float().clamp_min(6e-8)
    ls = (sub / d[:, None]).round().clamp(0, 31)
    eff = (d[:, None] * ls).clamp_min(1e-12)
    q = ((x / eff[..., None]).unsqueeze(-1) - kv).abs().argmin(-1)                  # [n, 8, 32]
    qs = (q[..., :16] | (q[..., 16:] << 4)).to(torch.uint8).reshape(n, 128)
    s6 = ls.long() + 32
    sl = (s6 & 0xF).view(n, 4, 2)
    scales_l = (sl[..., 0] | (sl[..., 1] << 4)).to(torch.uint8)
    sh = sum(((s6[:, i] >> 4) & 3) << (2 * i) for i in range(8))
    scales_h = torch.stack([sh & 0xFF, sh >> 8], -1).to(torch.uint8)
    return torch.cat([_f16_bytes(d), scales_h, scales_l, qs], 1)


def _d_iq4_xs(b):
    t = tables(b.device)
    n = b.shape[0]
    d = _bytes_f16(b[:, 0:2])
    sh = b[:, 2].long() | (b[:, 3].long() << 8)
    slb = b[:, 4:8].long()
    sl = torch.stack([slb & 0xF, slb >> 4], -1).reshape(n, 8)
    s6 = (sl | (torch.stack([(sh >> (2 * i)) & 3 for i in range(8)], 1) << 4)) - 32
    qs = b[:, 8:136].long().view(n, 8, 16)
    q = torch.cat([qs & 0xF, qs >> 4], -1)
    return ((d[:, None] * s6.float())[..., None] * t["iq4nl"][q]).reshape(n, QK_K)


_Q = {GGMLType.Q8_0: _q_q8_0, GGMLType.Q4_K: _q_q4_k, GGMLType.Q5_K: _q_q5_k, GGMLType.Q2_K: _q_q2_k,
      GGMLType.IQ2_XXS: _q_iq2_xxs, GGMLType.IQ3_XXS: _q_iq3_xxs, GGMLType.IQ1_M: _q_iq1_m, GGMLType.Q3_K: _q_q3_k,
      GGMLType.Q6_K: _q_q6_k, GGMLType.IQ2_XS: _q_iq2_xs, GGMLType.IQ4_XS: _q_iq4_xs}
_D = {GGMLType.Q8_0: _d_q8_0, GGMLType.Q4_K: _d_q4_k, GGMLType.Q5_K: _d_q5_k, GGMLType.Q2_K: _d_q2_k,
      GGMLType.IQ2_XXS: _d_iq2_xxs, GGMLType.IQ3_XXS: _d_iq3_xxs, GGMLType.IQ1_M: _d_iq1_m, GGMLType.Q3_K: _d_q3_k,
      GGMLType.Q6_K: _d_q6_k, GGMLType.IQ2_XS: _d_iq2_xs, GGMLType.IQ4_XS: _d_iq4_xs}


def quantize(w: torch.Tensor, t: GGMLType) -> torch.Tensor:
    """``w [rows, cols]`` -> raw blocks ``uint8 [rows, cols / block * block_bytes]``."""
    t = GGMLType(t)
    rows, cols = w.shape
    if t == GGMLType.F32:
        return w.float().contiguous().view(torch.uint8).reshape(rows, cols * 4)
    if t in (GGMLType.F16, GGMLType.BF16):
        dt = torch.float16 if t == GGMLType.F16 else torch.bfloat16
        return w.to(dt).contiguous().view(torch.uint8).reshape(rows, cols * 2)
    blocks = _Q[t](w)
    assert blocks.shape[1] == BLOCK_BYTES[t], (t, blocks.shape)
    return blocks.reshape(rows, cols // BLOCK_ELEMS[t] * BLOCK_BYTES[t]).contiguous()


def dequantize(raw: torch.Tensor, t: GGMLType, cols: int) -> torch.Tensor:
    """Raw blocks ``uint8 [rows, row_bytes]`` -> fp32 ``[rows, cols]`` (reference dequantisation)."""
    t = GGMLType(t)
    rows = raw.shape[0]
    if t == GGMLType.F32:
        return raw.contiguous().view(torch.float32).reshape(rows, cols)
    if t in (GGMLType.F16, GGMLType.BF16):
        dt = torch.float16 if t == GGMLType.F16 else torch.bfloat16
        return raw.contiguous().view(dt).reshape(rows, cols).float()
    return _D[t](raw.reshape(-1, BLOCK_BYTES[t])).reshape(rows, cols)
