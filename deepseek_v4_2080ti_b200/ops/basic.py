"""Row-wise kernels (csrc/kernels/elementwise.cu): norms, embedding, gating, conv, arg-max.

Each wrapper has an ``*_ref`` fp32 PyTorch oracle next to it.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

_ll = ctypes.c_longlong
_f = ctypes.c_float


def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6, unit_offset: bool = False,
            out: torch.Tensor | None = None) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * (gamma or 1 + gamma).  x: [rows, cols] bf16."""
    rows, cols = x.shape
    out = torch.empty_like(x) if out is None else out
    rc = _lib.lib().b200_rmsnorm(_lib.ptr(x), None, None, 0, _lib.ptr(gamma), _lib.ptr(out), _ll(rows), cols,
                                 _f(eps), int(unit_offset), 0, _lib.stream())
    _lib.check(rc, "rmsnorm")
    return out


def add_rmsnorm(resid: torch.Tensor, delta: torch.Tensor | None, gamma: torch.Tensor, eps: float = 1e-6,
                unit_offset: bool = False, partials: torch.Tensor | None = None, splits: int = 0,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """resid += delta (+ sum of fp32 split-K partials) in place; returns norm(resid)."""
    rows, cols = resid.shape
    out = torch.empty_like(resid) if out is None else out
    rc = _lib.lib().b200_rmsnorm(_lib.ptr(resid), _lib.ptr(delta), _lib.ptr(partials), splits, _lib.ptr(gamma),
                                 _lib.ptr(out), _ll(rows), cols, _f(eps), int(unit_offset), 1, _lib.stream())
    _lib.check(rc, "add_rmsnorm")
    return out


def rmsnorm_split(resid: torch.Tensor, delta: torch.Tensor | None, gamma: torch.Tensor, terms: int, eps: float = 1e-6,
                  unit_offset: bool = False, want_bf16: bool = True):
    """(resid += delta in place when delta is given) -> (norm(resid) bf16 or None, (xq, inv_c)): the norm output
    also as E4M3 terms for ``gemm.linear_stream`` (csrc/kernels/decode_fused.cu)."""
    rows, cols = resid.shape
    out = torch.empty_like(resid) if want_bf16 else None
    xq = torch.empty(rows * terms, cols, dtype=torch.uint8, device=resid.device)
    inv_c = torch.empty(rows, dtype=torch.float32, device=resid.device)
    rc = _lib.lib().b200_rmsnorm_split(_lib.ptr(resid), _lib.ptr(delta), _lib.ptr(gamma), _lib.ptr(out), _lib.ptr(xq),
                                       _lib.ptr(inv_c), rows, cols, _f(eps), int(unit_offset), terms, _lib.stream())
    _lib.check(rc, "rmsnorm_split")
    return out, (xq, inv_c)


def silu_mul_split(gu: torch.Tensor, terms: int):
    """gu [T, 2I] (gate | up) -> E4M3 terms of silu(gate) * up for ``gemm.linear_stream``: (xq [T*terms, I], inv_c [T])."""
    t, two_i = gu.shape
    inter = two_i // 2
    xq = torch.empty(t * terms, inter, dtype=torch.uint8, device=gu.device)
    inv_c = torch.empty(t, dtype=torch.float32, device=gu.device)
    rc = _lib.lib().b200_silu_mul_split(_lib.ptr(gu), _lib.ptr(xq), _lib.ptr(inv_c), t, inter, terms, _lib.stream())
    _lib.check(rc, "silu_mul_split")
    return xq, inv_c


def rmsnorm_ref(x, gamma, eps=1e-6, unit_offset=False):
    xf = x.float()
    g = gamma.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * (1 + g if unit_offset else g)


def gated_rmsnorm(x: torch.Tensor, gate: torch.Tensor, gamma: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """Per-head norm with SiLU gate.  x: [T, heads, dim] contiguous bf16 (dim <= 256);
    gate: same logical shape, last two dims contiguous, any row stride (a slice of a wider projection)."""
    dim = x.shape[-1]
    heads = x.shape[-2] if x.dim() >= 2 else 1
    gate_ld = gate.stride(0) if gate.dim() == 3 else heads * dim
    out = torch.empty_like(x)
    rc = _lib.lib().b200_gated_rmsnorm(_lib.ptr(x), _lib.ptr(gate), _lib.ptr(gamma), _lib.ptr(out),
                                       _ll(x.numel() // dim), dim, _f(eps), heads, _ll(gate_ld), _lib.stream())
    _lib.check(rc, "gated_rmsnorm")
    return out


def gated_rmsnorm_ref(x, gate, gamma, eps=1e-6):
    xf = x.float()
    return xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float() * F.silu(gate.float())


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_lo: int = 0, vocab_hi: int | None = None) -> torch.Tensor:
    """Rows of a (possibly vocab-sharded) table; ids outside [lo, hi) give zero rows."""
    hi = vocab_lo + table.shape[0] if vocab_hi is None else vocab_hi
    # ids of another shard give zero rows by design; negative ids or ids past the whole vocabulary are errors.  The
    # upper end is only known to the caller of a full table, so the check covers the unsharded case.
    if vocab_lo == 0 and vocab_hi is None:
        _lib.check_indices(ids if ids.dtype == torch.int32 and ids.is_contiguous() else None, 0, hi, 1)
    out = torch.empty(ids.numel(), table.shape[1], dtype=torch.bfloat16, device=table.device)
    rc = _lib.lib().b200_embedding(_lib.ptr(ids), _lib.ptr(table), _lib.ptr(out), ids.numel(), table.shape[1],
                                   vocab_lo, hi, _lib.stream())
    _lib.check(rc, "embedding")
    return out


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """gate_up: [rows, 2*I] (gate | up) -> silu(gate) * up [rows, I]."""
    rows, two_i = gate_up.shape
    inter = two_i // 2
    out = torch.empty(rows, inter, dtype=torch.bfloat16, device=gate_up.device)
    rc = _lib.lib().b200_silu_mul(_lib.ptr(gate_up), _lib.ptr(out), _ll(rows), inter, _lib.stream())
    _lib.check(rc, "silu_mul")
    return out


def silu_mul_ref(gate_up):
    g, u = gate_up.float().chunk(2, dim=-1)
    return F.silu(g) * u


def sigmoid_mul(x: torch.Tensor, gate: torch.Tensor) -> torch.Tensor:
    out = torch.empty_like(x)
    rc = _lib.lib().b200_sigmoid_mul(_lib.ptr(x), _lib.ptr(gate), _lib.ptr(out), _ll(x.numel()), _lib.stream())
    _lib.check(rc, "sigmoid_mul")
    return out


def add_(y: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    rc = _lib.lib().b200_add(_lib.ptr(y), _lib.ptr(x), _ll(y.numel()), _lib.stream())
    _lib.check(rc, "add")
    return y


def conv_silu(x: torch.Tensor, weight: torch.Tensor, tail: torch.Tensor, update_tail: bool = True) -> torch.Tensor:
    """Causal depthwise conv (kernel 4) + SiLU over x [T, C] (row stride allowed); tail [3, C] carries history."""
    t, c = x.shape
    y = torch.empty(t, c, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().b200_conv_silu(_lib.ptr(x), x.stride(0), _lib.ptr(weight), _lib.ptr(tail), _lib.ptr(y), c, t, c,
                                   weight.shape[-1], int(update_tail), _lib.stream())
    _lib.check(rc, "conv_silu")
    return y


def conv_silu_step(x: torch.Tensor, weight: torch.Tensor, tails: torch.Tensor, slot_ids: torch.Tensor | None) -> torch.Tensor:
    """One token per sequence; tails [slots, 3, C] updated in place."""
    b, c = x.shape
    y = torch.empty(b, c, dtype=torch.bfloat16, device=x.device)
    rc = _lib.lib().b200_conv_silu_step(_lib.ptr(x), x.stride(0), _lib.ptr(weight), _lib.ptr(tails),
                                        _ll(tails.stride(0)), _lib.ptr(slot_ids), _lib.ptr(y), c, b, c,
                                        weight.shape[-1], _lib.stream())
    _lib.check(rc, "conv_silu_step")
    return y


def conv_silu_ref(x, weight, tail):
    """x [T, C], weight [C, 4], tail [3, C] -> (y [T, C] fp32, new tail [3, C])."""
    kw = weight.shape[-1]
    full = torch.cat([tail.float(), x.float()], 0)  # [T+3, C]
    y = torch.zeros(x.shape[0], x.shape[1], dtype=torch.float32, device=x.device)
    for j in range(kw):
        y += full[j:j + x.shape[0]] * weight.float()[:, j]
    return F.silu(y), full[-(kw - 1):].to(x.dtype)


def gdn_gates(ab: torch.Tensor, a_off: int, b_off: int, a_log: torch.Tensor, dt_bias: torch.Tensor, heads: int):
    """g = -exp(A_log) * softplus(a + dt_bias), beta = sigmoid(b); a/b are column slices of ``ab`` [rows, ld]."""
    rows = ab.shape[0]
    g = torch.empty(rows, heads, dtype=torch.float32, device=ab.device)
    beta = torch.empty_like(g)
    rc = _lib.lib().b200_gdn_gates(_lib.ptr(ab), ab.stride(0), a_off, b_off, _lib.ptr(a_log), _lib.ptr(dt_bias),
                                   _lib.ptr(g), _lib.ptr(beta), _ll(rows), heads, _lib.stream())
    _lib.check(rc, "gdn_gates")
    return g, beta


def gdn_gates_ref(a, b, a_log, dt_bias):
    return -torch.exp(a_log.float()) * F.softplus(a.float() + dt_bias.float()), torch.sigmoid(b.float())


def argmax(logits: torch.Tensor, index_offset: int = 0, want_values: bool = False):
    rows, n = logits.shape
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device)
    val = torch.empty(rows, dtype=torch.float32, device=logits.device) if want_values else None
    rc = _lib.lib().b200_argmax(_lib.ptr(logits), int(logits.dtype == torch.float32), logits.stride(0), n, rows,
                                index_offset, _lib.ptr(idx), _lib.ptr(val), _lib.stream())
    _lib.check(rc, "argmax")
    return (idx, val) if want_values else idx
