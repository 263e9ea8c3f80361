"""FP8 E4M3 weights with one scale per 128x128 block.

Layout (same as the reference's checkpoints): ``W.weight`` float8_e4m3fn ``[out, in]`` and
``W.weight_scale_inv`` ``[ceil(out/128), ceil(in/128)]`` with ``w ~= fp8 * scale``
(cpp_engine/tests/qwen_parity_fixture.hpp:117-170, src/models/qwen4_exp/quant.py:59-95;
DeepSeek-style E8M0 ``scale`` tensors use the same geometry, src/models/deepseek_v4/runtime.py:650-760).
"""
from __future__ import annotations

import torch

FP8_MAX = 448.0
BLOCK = 128


def quantize_block128(w: torch.Tensor, scale_dtype=torch.bfloat16, pow2_scale: bool = False):
    """Quantize ``w [out, in]`` (any float dtype) -> (fp8 [out, in], scale [ceil(out/128), ceil(in/128)])."""
    out_f, in_f = w.shape
    ob, ib = (out_f + BLOCK - 1) // BLOCK, (in_f + BLOCK - 1) // BLOCK
    wp = torch.zeros(ob * BLOCK, ib * BLOCK, dtype=torch.float32, device=w.device)
    wp[:out_f, :in_f] = w.float()
    blocks = wp.view(ob, BLOCK, ib, BLOCK)
    amax = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / FP8_MAX
    if pow2_scale:
        scale = torch.exp2(torch.ceil(torch.log2(scale)))
    # the stored scale is what the kernels see: round it first, quantize against the rounded value
    scale = scale.to(scale_dtype).float()
    q = (blocks / scale[:, None, :, None]).clamp(-FP8_MAX, FP8_MAX)
    q = q.view(ob * BLOCK, ib * BLOCK)[:out_f, :in_f].contiguous().to(torch.float8_e4m3fn)
    return q, scale.to(scale_dtype)


def dequantize_block128(q: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """fp32 reference dequantisation."""
    out_f, in_f = q.shape
    s = scale.float().repeat_interleave(BLOCK, 0)[:out_f].repeat_interleave(BLOCK, 1)[:, :in_f]
    return q.float() * s
