"""ctypes front-ends of csrc/kernels/v4_ops.cu (Hadamard-128 rotation, hyper-connection mixers)."""
from __future__ import annotations

import ctypes

import torch

from . import _lib


def hadamard128(x: torch.Tensor) -> torch.Tensor:
    assert x.dtype == torch.bfloat16 and x.is_cuda and x.is_contiguous() and x.shape[-1] == 128
    y = torch.empty_like(x)
    rc = _lib.lib().b200_hadamard128(_lib.ptr(x), _lib.ptr(y), ctypes.c_longlong(x.numel() // 128), _lib.stream())
    _lib.check(rc, "hadamard128")
    return y


def hc_split_pre(mixes: torch.Tensor, x: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, iters: int, eps: float):
    """mixes fp32 [B, S, 24]; x bf16 [B, S, 4, D] -> (y bf16 [B, S, D], post fp32 [B, S, 4], comb fp32 [B, S, 4, 4])."""
    b, s, hc, d = x.shape
    assert hc == 4 and x.dtype == torch.bfloat16
    t = b * s
    y = torch.empty(b, s, d, dtype=torch.bfloat16, device=x.device)
    post = torch.empty(b, s, 4, dtype=torch.float32, device=x.device)
    comb = torch.empty(b, s, 4, 4, dtype=torch.float32, device=x.device)
    rc = _lib.lib().b200_hc_split_pre(_lib.ptr(mixes.float().contiguous()), _lib.ptr(x.contiguous()), _lib.ptr(scale.float().contiguous()),
                                      _lib.ptr(base.float().contiguous()), ctypes.c_longlong(t), d, iters, ctypes.c_float(eps),
                                      _lib.ptr(y), _lib.ptr(post), _lib.ptr(comb), _lib.stream())
    _lib.check(rc, "hc_split_pre")
    return y, post, comb


def hc_post(y: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    b, s, hc, d = residual.shape
    out = torch.empty_like(residual)
    rc = _lib.lib().b200_hc_post(_lib.ptr(y.contiguous()), _lib.ptr(residual.contiguous()), _lib.ptr(post.float().contiguous()),
                                 _lib.ptr(comb.float().contiguous()), ctypes.c_longlong(b * s), d, _lib.ptr(out), _lib.stream())
    _lib.check(rc, "hc_post")
    return out
