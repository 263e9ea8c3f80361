"""GQA attention over a paged KV cache (head_dim 128): fused q/k norm + partial RoPE + cache
append, tcgen05 flash prefill, split-context decode.  Cache layout:
``[num_blocks, kv_heads, block_size, 128]`` bf16, zero-initialised.
"""
from __future__ import annotations

import ctypes
import math

import torch

from . import _lib

_f = ctypes.c_float
D = 128


def rope_inv_freq(rot: int, theta: float, device) -> torch.Tensor:
    return (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float64) / rot))).float().to(device)


def qk_norm_rope_append(q_src, q_off, q_head_stride, gate_in_q, k_src, k_off, v_src, v_off, q_gamma, k_gamma,
                        unit_offset, eps, inv_freq, rot, positions, slots, k_cache, v_cache, n_q_heads, n_kv_heads,
                        mscale: float = 1.0):
    """Normalise + rotate q and k, split the q||gate layout, and write K/V rows into the paged cache.

    ``*_src`` are 2-D bf16 tensors (often the same fused-projection output) addressed as
    ``src[t, off + head * stride + d]``. Returns (q [T, Hq, 128], gate [T, Hq, 128] or None).
    """
    t = q_src.shape[0]
    bs = k_cache.shape[2]
    _lib.check_indices(slots, 0, k_cache.shape[0] * bs, 2)
    q_out = torch.empty(t, n_q_heads, D, dtype=torch.bfloat16, device=q_src.device)
    gate_out = torch.empty_like(q_out) if gate_in_q else None
    rc = _lib.lib().b200_qk_norm_rope_append(
        _lib.ptr(q_src), q_src.stride(0), q_off, q_head_stride, int(gate_in_q),
        _lib.ptr(k_src), k_src.stride(0), k_off, _lib.ptr(v_src), v_src.stride(0), v_off,
        _lib.ptr(q_gamma), _lib.ptr(k_gamma), int(unit_offset), _f(eps), _lib.ptr(inv_freq), rot, _f(mscale),
        _lib.ptr(positions), _lib.ptr(slots), _lib.ptr(q_out), _lib.ptr(gate_out), _lib.ptr(k_cache),
        _lib.ptr(v_cache), bs, t, n_q_heads, n_kv_heads, _lib.stream())
    _lib.check(rc, "qk_norm_rope_append")
    return q_out, gate_out


def qk_sumsq(proj: torch.Tensor, q_off: int, q_width: int, k_off: int, k_width: int) -> torch.Tensor:
    """fp32 [T, 2]: sums of squares of the q and k column ranges of each projection row."""
    t = proj.shape[0]
    out = torch.empty(t, 2, dtype=torch.float32, device=proj.device)
    rc = _lib.lib().b200_qk_sumsq(_lib.ptr(proj), proj.stride(0), q_off, q_width, k_off, k_width, _lib.ptr(out), t, _lib.stream())
    _lib.check(rc, "qk_sumsq")
    return out


def qk_fullnorm_rope_append(proj, q_off, k_off, v_off, q_gamma, k_gamma, row_ss, q_full_width, k_full_width, eps, inv_freq,
                            rot, positions, slots, k_cache, v_cache, n_q_heads, n_kv_heads):
    """MiniMax-style attention prologue: RMSNorm whose statistic spans the whole q / k projection row (``row_ss`` holds
    the rows' sums of squares over all ranks), per-(head, dim) gamma, half-split partial RoPE, paged K/V append."""
    t = proj.shape[0]
    bs = k_cache.shape[2]
    q_out = torch.empty(t, n_q_heads, D, dtype=torch.bfloat16, device=proj.device)
    rc = _lib.lib().b200_qk_fullnorm_rope_append(
        _lib.ptr(proj), proj.stride(0), q_off, _lib.ptr(proj), proj.stride(0), k_off, _lib.ptr(proj), proj.stride(0), v_off,
        _lib.ptr(q_gamma), _lib.ptr(k_gamma), _lib.ptr(row_ss), q_full_width, k_full_width, _f(eps), _lib.ptr(inv_freq), rot,
        _lib.ptr(positions), _lib.ptr(slots), _lib.ptr(q_out), _lib.ptr(k_cache), _lib.ptr(v_cache), bs, t, n_q_heads,
        n_kv_heads, _lib.stream())
    _lib.check(rc, "qk_fullnorm_rope_append")
    return q_out


def prefill(q, k_cache, v_cache, block_table, q_start, q_len, kv_len, max_q_len, gate=None, scale=None, window: int = 0,
            sinks: int = 0):
    """Causal attention of new query rows against the paged cache (which already holds their K/V).

    q: [T, Hq, 128]; block_table [B, max_blocks] int32; q_start/q_len/kv_len [B] int32 device tensors.
    """
    t, hq, d = q.shape
    assert d == D
    nb, hkv, bs, _ = k_cache.shape
    _lib.check_indices(block_table, 0, nb, 3)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    rc = _lib.lib().b200_gqa_prefill_ex(
        _lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(out), _lib.ptr(gate), _lib.ptr(block_table),
        _lib.ptr(q_start), _lib.ptr(q_len), _lib.ptr(kv_len), block_table.shape[0], int(max_q_len), t,
        block_table.shape[1], nb, bs, hq, hkv, _f(scale), int(window), int(sinks), _lib.ptr(_lib.status_word(q.device)),
        _lib.stream())
    _lib.check(rc, "gqa_prefill")
    return out


_dec_ws: dict[int, torch.Tensor] = {}


def decode(q, k_cache, v_cache, block_table, kv_len, gate=None, scale=None, splits: int | None = None,
           max_kv_len: int | None = None, window: int = 0, sinks: int = 0):
    """One query row per sequence. q: [B, Hq, 128].  ``window`` > 0: only the first ``sinks`` and the last ``window``
    keys of each sequence are visible (sliding window with attention sinks)."""
    b, hq, d = q.shape
    nb, hkv, bs, _ = k_cache.shape
    _lib.check_indices(block_table, 0, nb, 3)
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if splits is None:
        ctx = max_kv_len if max_kv_len is not None else block_table.shape[1] * bs
        splits = max(1, min(64, (2 * 148) // max(1, b * hkv), (ctx + 255) // 256))
    ws = None
    if splits > 1:
        need = b * hq * splits * (D + 2)
        dev = q.device.index or 0
        ws = _dec_ws.get(dev)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
            _dec_ws[dev] = ws
    rc = _lib.lib().b200_gqa_decode_ex(_lib.ptr(q), _lib.ptr(k_cache), _lib.ptr(v_cache), _lib.ptr(out), _lib.ptr(gate),
                                       _lib.ptr(block_table), _lib.ptr(kv_len), _lib.ptr(ws), b, block_table.shape[1],
                                       bs, hq, hkv, splits, _f(scale), int(window), int(sinks), _lib.stream())
    _lib.check(rc, "gqa_decode", 2 if splits > 1 else 1)
    return out


# ---------------------------------------------------------------- quantised KV cache
KV8_FORMATS = {"fp8": 1, "int8_per_token_head": 2, "turboquant_k8v4": 3}


class Kv8Cache:
    """Quantised paged cache of one attention layer set: ``fmt`` "fp8" = E4M3 keys and values, "int8_per_token_head" =
    INT8, "turboquant_k8v4" = E4M3 keys + 4-bit affine values.  ``k`` uint8 [L, num_blocks, Hkv, bs, 128], ``v`` the
    same (64 bytes per row for 4-bit values), one fp32 scale per (block, head, row) in ``k_scale`` / ``v_scale``
    [L, num_blocks, Hkv, bs] and, for 4-bit values, the row minimum in ``v_min``.  Rows reach it through a bf16
    staging cache (the fused norm + RoPE kernel writes there) and ``kv8_quantize``."""

    def __init__(self, fmt: str, layers: int, num_blocks: int, hkv: int, block_size: int, device):
        self.fmt = KV8_FORMATS[fmt]
        self.k = torch.zeros(layers, num_blocks, hkv, block_size, D, dtype=torch.uint8, device=device)
        self.v = torch.zeros(layers, num_blocks, hkv, block_size, D // 2 if self.fmt == 3 else D, dtype=torch.uint8,
                             device=device)
        self.k_scale = torch.zeros(layers, num_blocks, hkv, block_size, dtype=torch.float32, device=device)
        self.v_scale = torch.zeros_like(self.k_scale)
        self.v_min = torch.zeros_like(self.k_scale) if self.fmt == 3 else None

    def layer(self, idx: int):
        """(k, v, k_scale, v_scale, v_min) views of one layer."""
        return self.k[idx], self.v[idx], self.k_scale[idx], self.v_scale[idx], None if self.v_min is None else self.v_min[idx]

    def nbytes(self) -> int:
        return self.k.numel() + self.v.numel() + 4 * self.k_scale.numel() * (3 if self.fmt == 3 else 2)


def kv8_quantize(fmt: int, stage_k, stage_v, src_slots, dst_slots, k8, v8, k_scale, v_scale, v_min=None):
    """Quantise staged rows ``src_slots`` (bf16 [nb_s, Hkv, bs_s, 128]) into rows ``dst_slots`` of the cache."""
    rc = _lib.lib().b200_kv8_quantize(_lib.ptr(stage_k), _lib.ptr(stage_v), _lib.ptr(src_slots), _lib.ptr(dst_slots),
                                      _lib.ptr(k8), _lib.ptr(v8), _lib.ptr(k_scale), _lib.ptr(v_scale), _lib.ptr(v_min),
                                      stage_k.shape[2], k8.shape[2], src_slots.numel(), k8.shape[1], int(fmt), _lib.stream())
    _lib.check(rc, "kv8_quantize")


def kv8_dequantize(fmt: int, k8, v8, k_scale, v_scale, block_table_row, n_tokens: int, stage_k, stage_v, v_min=None):
    """Dequantise the first ``n_tokens`` positions of one sequence into the staging caches (blocks 0, 1, 2, ...)."""
    if n_tokens <= 0:
        return
    assert stage_k.shape[2] == k8.shape[2] and stage_k.shape[0] * stage_k.shape[2] >= n_tokens
    rc = _lib.lib().b200_kv8_dequantize(_lib.ptr(k8), _lib.ptr(v8), _lib.ptr(k_scale), _lib.ptr(v_scale), _lib.ptr(v_min),
                                        _lib.ptr(block_table_row), _lib.ptr(stage_k), _lib.ptr(stage_v), k8.shape[2],
                                        int(n_tokens), k8.shape[1], int(fmt), _lib.stream())
    _lib.check(rc, "kv8_dequantize")


def decode_kv8(fmt: int, q, k8, v8, k_scale, v_scale, block_table, kv_len, gate=None, scale=None, splits: int | None = None,
               max_kv_len: int | None = None, window: int = 0, sinks: int = 0, v_min=None):
    """``decode`` over a quantised cache; rows are dequantised in registers."""
    b, hq, d = q.shape
    nb, hkv, bs, _ = k8.shape
    out = torch.empty_like(q)
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    if splits is None:
        ctx = max_kv_len if max_kv_len is not None else block_table.shape[1] * bs
        splits = max(1, min(64, (2 * 148) // max(1, b * hkv), (ctx + 255) // 256))
    ws = None
    if splits > 1:
        need = b * hq * splits * (D + 2)
        dev = q.device.index or 0
        ws = _dec_ws.get(dev)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
            _dec_ws[dev] = ws
    rc = _lib.lib().b200_gqa_decode_kv8(int(fmt), _lib.ptr(q), _lib.ptr(k8), _lib.ptr(v8), _lib.ptr(k_scale),
                                        _lib.ptr(v_scale), _lib.ptr(v_min), _lib.ptr(out), _lib.ptr(gate), _lib.ptr(block_table),
                                        _lib.ptr(kv_len), _lib.ptr(ws), b, block_table.shape[1], bs, hq, hkv, splits,
                                        _f(scale), int(window), int(sinks), _lib.stream())
    _lib.check(rc, "gqa_decode_kv8", 2 if splits > 1 else 1)
    return out


# ---------------------------------------------------------------- fp32 oracles
def rope_ref(x, positions, inv_freq, rot):
    """Half-split rotation over the first ``rot`` dims. x: [T, H, D] fp32."""
    half = rot // 2
    ang = positions.double()[:, None] * inv_freq.double()[None, :]
    cos, sin = ang.cos().float()[:, None, :], ang.sin().float()[:, None, :]
    a, b = x[..., :half], x[..., half:rot]
    return torch.cat([a * cos - b * sin, b * cos + a * sin, x[..., rot:]], -1)


def attention_ref(q, k, v, causal_offset: int, gate=None, scale=None):
    """q [Tq, Hq, D], k/v [Tk, Hkv, D] fp32; query i sees keys <= causal_offset + i."""
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    g = hq // hkv
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    kk = k.float().repeat_interleave(g, 1)
    vv = v.float().repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q.float(), kk) * scale
    mask = torch.arange(tk, device=q.device)[None, :] > (causal_offset + torch.arange(tq, device=q.device))[:, None]
    s = s.masked_fill(mask[None], float("-inf"))
    o = torch.einsum("hqk,khd->qhd", s.softmax(-1), vv)
    if gate is not None:
        o = o * torch.sigmoid(gate.float())
    return o
