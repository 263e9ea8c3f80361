"""Gated DeltaNet kernels (csrc/kernels/gdn.cu): chunked scan for prefill, single step for decode."""
from __future__ import annotations

import ctypes

import torch

from ..utils import canary
from . import _lib

_ll = ctypes.c_longlong
_ws: dict[int, torch.Tensor] = {}


def _workspace(n: int, device) -> torch.Tensor:
    dev = torch.device(device).index or 0
    ws = _ws.get(dev)
    if ws is None or ws.numel() < n:
        ws = canary.empty(n, dtype=torch.float32, device=device, name="gdn chunk operands")
        _ws[dev] = ws
    return ws


def chunked(mixed, q_off, k_off, v_off, g, beta, state, hv, hk):
    """mixed [T, ld] bf16 (q|k|v after conv), g/beta [T, Hv] fp32, state [Hv,128,128] fp32 (in place)."""
    t = mixed.shape[0]
    out = torch.empty(t, hv, 128, dtype=torch.bfloat16, device=mixed.device)
    L = _lib.lib()
    L.b200_gdn_workspace_floats.restype = ctypes.c_longlong
    ws = _workspace(int(L.b200_gdn_workspace_floats(t, hv)), mixed.device)
    rc = L.b200_gdn_chunked(_lib.ptr(mixed), mixed.stride(0), q_off, k_off, v_off, _lib.ptr(g), _lib.ptr(beta),
                            _lib.ptr(state), _lib.ptr(out), _lib.ptr(ws), t, hv, hk, _lib.stream())
    _lib.check(rc, "gdn_chunked", 2)
    return out


def use_simt_prepare(on: bool) -> bool:
    """Route the chunk preparation of ``chunked`` through the scalar fp32 kernel (the yardstick of the tensor-core
    one); returns the previous setting."""
    return bool(_lib.lib().b200_gdn_use_simt_prepare(int(bool(on))))


def step(states, slot_ids, mixed, q_off, k_off, v_off, g, beta, hv, hk):
    """states [slots, Hv, 128, 128] fp32 in place; mixed [B, ld]; returns [B, Hv, 128] bf16."""
    b = mixed.shape[0]
    out = torch.empty(b, hv, 128, dtype=torch.bfloat16, device=mixed.device)
    _lib.check_indices(slot_ids, 0, states.shape[0], 4)
    rc = _lib.lib().b200_gdn_step(_lib.ptr(states), _ll(states.stride(0)), _lib.ptr(slot_ids), _lib.ptr(mixed),
                                  mixed.stride(0), q_off, k_off, v_off, _lib.ptr(g), _lib.ptr(beta), _lib.ptr(out),
                                  b, hv, hk, _lib.stream())
    _lib.check(rc, "gdn_step")
    return out


def decode_fused(proj, x, w_ab, a_log, dt_bias, conv_w, tails, states, slot_ids, gamma, hv, hk, eps=1e-6):
    """Whole Gated-DeltaNet token mixer of a decode step in one launch (csrc/kernels/decode_fused.cu).

    proj [B, 2kd+2vd] bf16 = q|k|v|z projection output; x [B, hidden] bf16 normed layer input; w_ab [2Hv, hidden]
    bf16 (a rows, then b rows); conv_w [2kd+vd, 4] bf16; tails [slots, 3, 2kd+vd] bf16 and states
    [slots, Hv, 128, 128] fp32 are updated in place for ``slot_ids`` (int32 [B]).  Returns [B, Hv*128] bf16
    (gated-RMSNorm output, the input of the output projection)."""
    b = proj.shape[0]
    _lib.check_indices(slot_ids, 0, states.shape[0], 4)
    out = torch.empty(b, hv * 128, dtype=torch.bfloat16, device=proj.device)
    rc = _lib.lib().b200_gdn_decode_fused(
        _lib.ptr(proj), proj.stride(0), _lib.ptr(x), x.shape[1], _lib.ptr(w_ab), _lib.ptr(a_log), _lib.ptr(dt_bias),
        _lib.ptr(conv_w), conv_w.shape[1], _lib.ptr(tails), _ll(tails.stride(0)), _lib.ptr(states),
        _ll(states.stride(0)), _lib.ptr(slot_ids), _lib.ptr(gamma), _lib.ptr(out), b, hv, hk, ctypes.c_float(eps),
        _lib.stream())
    _lib.check(rc, "gdn_decode_fused")
    return out


def recurrent_ref(q, k, v, g, beta, state):
    """fp32 oracle, token by token. q,k [T,Hk,128]; v [T,Hv,128]; g,beta [T,Hv]; state [Hv,128,128] (dk, dv).

    Same recurrence as the reference's step kernel (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:2282-2347).
    """
    t, hk, dk = q.shape
    hv = v.shape[1]
    rep = hv // hk
    qf = q.float()
    kf = k.float()
    qf = qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    kf = kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)
    qf = qf.repeat_interleave(rep, 1)
    kf = kf.repeat_interleave(rep, 1)
    s = state.float().clone()
    outs = []
    for i in range(t):
        s = s * torch.exp(g[i].float())[:, None, None]
        kv_mem = torch.einsum("hkv,hk->hv", s, kf[i])
        delta = (v[i].float() - kv_mem) * beta[i].float()[:, None]
        s = s + kf[i][:, :, None] * delta[:, None, :]
        outs.append(torch.einsum("hkv,hk->hv", s, qf[i]))
    return torch.stack(outs), s
