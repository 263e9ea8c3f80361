"""Sparse-selected grouped-query attention (Qwen4-Exp "QSA" layers) on the GPU.

Every query token attends only to the tokens its indexer picked (``sel`` [S, W] int32, -1 = empty; the same list for
all heads).  The gather-based tensor-core kernel of the latent-attention family does the work
(csrc/kernels/attn_mla_mma.cu, instantiated for 256-wide rows): the cache keeps one row per (kv head, token) laid out
``[value (128) | key (128)]``; a query is presented as ``[0 | q]``, so the score is ``q . key`` and the output
``P . value``.  The kv heads become extra "tokens" of the launch (S x Hkv of them, each with its group of
H / Hkv query heads as the M dimension of the MMAs) addressing their own run of cache pages, which keeps the whole
layer one launch plus a transpose.

Reference: ``cuda_qsa_attention`` (src/csrc/qwen4_exp_qsa.cu:69,288) and its torch fallback
(src/models/qwen4_exp/attention.py:655-720); the selection itself is ``qsa_select`` in
models/qwen4_exp_components.py, plain tensor code that runs on either device.
"""
from __future__ import annotations

import math

import torch

from . import _lib, mla

D = 128
BLOCK = 64


class QsaCache:
    """[Hkv, capacity, 256] bf16 rows (value | key) and the page table that gives every kv head its own run of pages."""

    def __init__(self, n_kv_heads: int, capacity: int, device):
        self.hkv = n_kv_heads
        self.capacity = (capacity + BLOCK - 1) // BLOCK * BLOCK
        self.rows = torch.zeros(n_kv_heads, self.capacity, 2 * D, dtype=torch.bfloat16, device=device)
        nblk = self.capacity // BLOCK
        self.block_table = (torch.arange(n_kv_heads, device=device, dtype=torch.int32).view(-1, 1) * nblk +
                            torch.arange(nblk, device=device, dtype=torch.int32).view(1, -1)).contiguous()
        self.length = 0

    def append(self, k: torch.Tensor, v: torch.Tensor) -> int:
        """k, v [S, Hkv, 128] (k normalised and rotated) for positions [length, length + S); returns the old length."""
        s = k.shape[0]
        past = self.length
        if past + s > self.capacity:
            raise ValueError(f"QSA cache holds {self.capacity} tokens; {past + s} needed")
        self.rows[:, past:past + s, :D] = v.transpose(0, 1)
        self.rows[:, past:past + s, D:] = k.transpose(0, 1)
        self.length = past + s
        return past


def attention(q: torch.Tensor, cache: QsaCache, sel: torch.Tensor, positions: torch.Tensor, scale: float | None = None
              ) -> torch.Tensor:
    """q [S, H, 128] bf16, sel [S, W] int32 token positions (-1 = empty), positions [S] int32 -> o [S, H, 128] bf16."""
    s, h, d = q.shape
    assert d == D and h % cache.hkv == 0 and q.dtype == torch.bfloat16
    hkv, g = cache.hkv, h // cache.hkv
    scale = 1.0 / math.sqrt(D) if scale is None else scale
    t = s * hkv
    dev = q.device
    q_pe = q.contiguous().view(t, g, D)                                  # virtual token (s, j): heads j*g .. j*g + g - 1
    q_lat = torch.zeros(g, t, D, dtype=torch.bfloat16, device=dev)
    sel_v = sel.to(torch.int32).repeat_interleave(hkv, dim=0).contiguous()             # the same list for every kv head
    pos_v = positions.to(torch.int32).repeat_interleave(hkv).contiguous()
    seq_v = torch.arange(hkv, dtype=torch.int32, device=dev).repeat(s).contiguous()    # page-table row = kv head
    o = mla.attention(q_lat, q_pe, cache.rows.view(-1, 2 * D), cache.block_table, BLOCK, pos_v, D, D, scale, sel=sel_v,
                      seq_of_token=seq_v)                                              # [g, t, 128]
    return mla.transpose_heads(o).view(s, hkv * g, D)


def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, sel: torch.Tensor, scale: float | None = None
                  ) -> torch.Tensor:
    """fp32 statement: q [S, H, D], k / v [L, Hkv, D], sel [S, W] -> [S, H, D]."""
    s, h, d = q.shape
    hkv = k.shape[1]
    scale = 1.0 / math.sqrt(d) if scale is None else scale
    safe = sel.clamp_min(0).long()
    gk, gv = k.float()[safe], v.float()[safe]                            # [S, W, Hkv, D]
    qh = q.float().view(s, hkv, h // hkv, d)
    sc = torch.einsum("qkgd,qskd->qkgs", qh, gk) * scale
    sc = sc.masked_fill((sel < 0)[:, None, None, :], float("-inf"))
    return torch.einsum("qkgs,qskd->qkgd", sc.softmax(-1), gv).reshape(s, h, d)
