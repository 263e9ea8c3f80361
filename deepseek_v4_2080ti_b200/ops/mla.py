"""Latent-attention kernels (csrc/kernels/attn_mla.cu): cache append, query preparation, indexer scores, row top-k,
sparse absorbed attention, head transposes, and the per-head (grouped) absorption GEMMs."""
from __future__ import annotations

import ctypes

import torch

from . import _lib, gemm

_f = ctypes.c_float


def kv_append(kv, gamma, eps, positions, slots, theta, cache, c, r, kidx=None, kidx_gamma=None, idx_cache=None):
    """kv [T, c + r] bf16 -> cache rows ``slots`` [T] (normalised latent | rotated key); optional indexer keys."""
    _lib.check_indices(slots, 0, cache.shape[0], 2)
    t = kv.shape[0]
    di = kidx.shape[1] if kidx is not None else 0
    rc = _lib.lib().b200_mla_kv_append(_lib.ptr(kv), _lib.ptr(gamma), _f(eps), _lib.ptr(positions), _lib.ptr(slots), _f(theta),
                                       _lib.ptr(cache), t, c, r, _lib.ptr(kidx), _lib.ptr(kidx_gamma), _lib.ptr(idx_cache), di,
                                       _lib.stream())
    _lib.check(rc, "mla_kv_append")


def q_prepare(q, positions, theta, h, n, r):
    """q [T, h*(n + r)] -> (q_nope transposed [h, T, n], rotated q_pe [T, h, r])."""
    t = q.shape[0]
    qn = torch.empty(h, t, n, dtype=torch.bfloat16, device=q.device)
    qp = torch.empty(t, h, r, dtype=torch.bfloat16, device=q.device)
    rc = _lib.lib().b200_mla_q_prepare(_lib.ptr(q), _lib.ptr(positions), _f(theta), _lib.ptr(qn), _lib.ptr(qp), t, h, n, r,
                                       _lib.stream())
    _lib.check(rc, "mla_q_prepare")
    return qn, qp


def indexer_scores(q_idx, hw, idx_cache, block_table, bs, positions, ld, scale, seq_of_token=None):
    """q_idx [T, HI, DI] bf16, hw [T, HI] fp32 -> scores fp32 [T, ld] (-inf beyond each row's position)."""
    t, hi, di = q_idx.shape
    scores = torch.empty(t, ld, dtype=torch.float32, device=q_idx.device)
    rc = _lib.lib().b200_mla_indexer(_lib.ptr(q_idx), _lib.ptr(hw), _lib.ptr(idx_cache), _lib.ptr(block_table),
                                     block_table.shape[-1], bs, _lib.ptr(positions), _lib.ptr(seq_of_token), _lib.ptr(scores),
                                     ld, t, hi, di, _f(scale), _lib.stream())
    _lib.check(rc, "mla_indexer")
    return scores


def topk_rows(vals: torch.Tensor, n_valid: torch.Tensor, k: int) -> torch.Tensor:
    """Indices of the k largest of the first n_valid[row] entries of every row; -1 padding; unordered."""
    rows, ld = vals.shape
    idx = torch.empty(rows, k, dtype=torch.int32, device=vals.device)
    rc = _lib.lib().b200_topk_rows(_lib.ptr(vals), ld, _lib.ptr(n_valid), rows, k, _lib.ptr(idx), _lib.stream())
    _lib.check(rc, "topk_rows")
    return idx


_split_ws: dict[int, torch.Tensor] = {}


def attention(q_lat, q_pe, cache, block_table, bs, positions, c, r, scale, sel=None, seq_of_token=None, max_keys: int | None = None,
              splits: int | None = None):
    """q_lat [H, T, c], q_pe [T, H, r] -> o_lat [H, T, c]; ``sel`` [T, nsel] int32 cache positions or None (dense causal).
    With few query tokens (decode) the context is split over several CTAs per head group (``splits``; chosen from the
    grid size and ``max_keys``, an upper bound of the keys a token attends to) and merged by a second kernel."""
    h, t, _ = q_lat.shape
    # selected positions address the sequence's pages: [0, pages * block) with -1 = no entry; page ids address the cache
    _lib.check_indices(sel, 0, block_table.shape[-1] * bs, 5, keep=-1)
    _lib.check_indices(block_table, 0, max(1, cache.shape[0] // bs), 3)          # cache [rows, c + r]: rows / block pages
    o = torch.empty(h, t, c, dtype=torch.bfloat16, device=q_lat.device)
    groups = t * ((h + 15) // 16)
    if splits is None:
        nk = sel.shape[1] if sel is not None else (max_keys if max_keys is not None else block_table.shape[-1] * bs)
        splits = 1 if groups >= 148 else max(1, min(32, 296 // groups, (nk + 63) // 64))
    ws = None
    if splits > 1:
        need = t * h * splits * (c + 2)
        dev = q_lat.device.index or 0
        ws = _split_ws.get(dev)
        if ws is None or ws.numel() < need:
            ws = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q_lat.device)
            _split_ws[dev] = ws
    rc = _lib.lib().b200_mla_attention_splitkv(_lib.ptr(q_lat), _lib.ptr(q_pe), _lib.ptr(cache), _lib.ptr(block_table),
                                               block_table.shape[-1], bs, _lib.ptr(positions), _lib.ptr(seq_of_token),
                                               _lib.ptr(sel), 0 if sel is None else sel.shape[1], _lib.ptr(o), t, h, c, r,
                                               _f(scale), _lib.ptr(ws), int(splits), _lib.stream())
    _lib.check(rc, "mla_attention", 2 if splits > 1 else 1)
    return o


def transpose_heads(x):
    """[H, T, D] -> [T, H, D]."""
    h, t, d = x.shape
    out = torch.empty(t, h, d, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().b200_transpose_heads(_lib.ptr(x), _lib.ptr(out), h, t, d, _lib.stream())
    _lib.check(rc, "transpose_heads")
    return out


_uniform_tables: dict[tuple, tuple[torch.Tensor, torch.Tensor, int]] = {}


def per_head_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [H, T, K] bf16, w [H*N, K] bf16 (head h uses rows h*N..): y[h] = x[h] @ w[h]^T -> [H, T, N].
    One grouped tcgen05 GEMM over a fixed work table (every head has T rows); N % 128 == 0, K % 16 == 0."""
    h, t, k = x.shape
    n = w.shape[0] // h
    bn = gemm._bn(t)
    key = (h, t, n, bn, x.device.index)
    tab = _uniform_tables.get(key)
    if tab is None:
        mt, nt = n // 128, (t + bn - 1) // bn
        g = torch.arange(h).view(h, 1, 1).expand(h, nt, mt)
        tn = torch.arange(nt).view(1, nt, 1).expand(h, nt, mt)
        m = torch.arange(mt).view(1, 1, mt).expand(h, nt, mt)
        rows = torch.clamp(t - tn * bn, max=bn)
        work = torch.stack([g, m, g * t + tn * bn, rows], -1).reshape(-1, 4).to(torch.int32).to(x.device)
        tab = (work.contiguous(), torch.tensor([work.shape[0]], dtype=torch.int32, device=x.device), bn)
        _uniform_tables[key] = tab
    work, nwork, bn = tab
    out = torch.empty(h, t, n, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().b200_gemm_wdec_grouped(gemm.WF_BF16, _lib.ptr(w), None, _lib.ptr(x), _lib.ptr(out), h * t, n, k, h,
                                           _lib.ptr(work), _lib.ptr(nwork), bn, _lib.ptr(_lib.status_word(x.device)),
                                           _lib.stream())
    _lib.check(rc, "per_head_linear")
    return out
