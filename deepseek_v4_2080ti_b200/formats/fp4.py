"""FP4 E2M1 weights with one UE8M0 (power-of-two) scale per 32 consecutive input elements.

Layout (DeepSeek routed experts): ``weight`` uint8 ``[out, in/2]`` holding two 4-bit codes per byte,
**low nibble first**, and ``scale`` uint8 ``[out, in/32]`` holding the biased exponent e of 2^(e-127).
A code is sign (bit 3) plus a 3-bit index into {0, 0.5, 1, 1.5, 2, 3, 4, 6}
(reference: src/kernels/ops.py:110-155, cpp_engine/backends/cuda/kernels/fp4_ops.cu:33-36).
"""
from __future__ import annotations

import torch

GROUP = 32
LEVELS = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
FP4_MAX = 6.0


def level_table(device="cpu") -> torch.Tensor:
    """16-entry value table indexed by the 4-bit code."""
    pos = torch.tensor(LEVELS, dtype=torch.float32, device=device)
    return torch.cat([pos, -pos])


def quantize(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """``w [out, in]`` (in % 32 == 0) -> (packed uint8 [out, in/2], e8m0 uint8 [out, in/32])."""
    out_f, in_f = w.shape
    assert in_f % GROUP == 0
    g = w.float().view(out_f, in_f // GROUP, GROUP)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -120)
    # smallest power of two with amax / scale <= 6
    e = torch.ceil(torch.log2(amax / FP4_MAX)).clamp(-127, 127)
    scale = torch.exp2(e)
    y = (g / scale[..., None]).clamp(-FP4_MAX, FP4_MAX)
    pos = torch.tensor(LEVELS, dtype=torch.float32, device=w.device)
    idx = (y.abs()[..., None] - pos).abs().argmin(-1).to(torch.uint8)
    code = idx | ((y < 0) & (idx > 0)).to(torch.uint8) << 3
    code = code.view(out_f, in_f)
    packed = (code[:, 0::2] | (code[:, 1::2] << 4)).contiguous()
    return packed, (e + 127).to(torch.uint8).contiguous()


def unpack_codes(packed: torch.Tensor) -> torch.Tensor:
    out_f, half = packed.shape
    codes = torch.empty(out_f, half * 2, dtype=torch.uint8, device=packed.device)
    codes[:, 0::2] = packed & 0x0F
    codes[:, 1::2] = packed >> 4
    return codes


def dequantize(packed: torch.Tensor, scale_e8m0: torch.Tensor) -> torch.Tensor:
    """fp32 reference dequantisation of (packed, e8m0) -> [out, in]."""
    vals = level_table(packed.device)[unpack_codes(packed).long()]
    s = torch.exp2(scale_e8m0.float() - 127.0).repeat_interleave(GROUP, 1)
    return vals * s
