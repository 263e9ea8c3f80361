"""NVFP4 weights as the Qwen NVFP4 checkpoints hold them: E2M1 values packed two per byte (low nibble first), one E4M3
scale per 16 consecutive input channels, one fp32 global scale per tensor; value = e2m1 * e4m3_scale / global_scale.
Also the 36-byte ``Block64`` record (four group scales, then the 32 bytes of 64 values) the reference's native runtime
keeps on the device.

Reference behaviour: docs/models/qwen3.8-27b-nvfp4.md:30-46 (numerics and the record), cpp_engine/core/
qwen_weight_map.cpp:648-652 (tensor names ``.weight_packed`` / ``.weight_scale`` / ``.weight_global_scale`` /
``.input_global_scale``), qwen_nvfp4_ops.cu nvfp4_group16_reference :629.  This runtime expands such matrices to bf16
once at load and multiplies them on the bf16 tensor-core path: every NVFP4 value (a 1-bit mantissa times a 3-bit
mantissa scale) is exact in bf16 before the global scale."""
from __future__ import annotations

import torch

E2M1_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)
GROUP = 16


def _lut(device) -> torch.Tensor:
    pos = torch.tensor(E2M1_VALUES, dtype=torch.float32, device=device)
    return torch.cat([pos, -pos])                      # code bit 3 is the sign


def quantize(w: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """fp32 / bf16 [N, K] (K % 16 == 0) -> (weight_packed uint8 [N, K/2], weight_scale float8_e4m3fn [N, K/16],
    weight_global_scale fp32 [1]).  The global scale maps the largest group scale onto the E4M3 maximum."""
    w = w.float()
    n, k = w.shape
    assert k % GROUP == 0
    g = w.view(n, k // GROUP, GROUP)
    amax = g.abs().amax(-1)                                                   # [N, K/16]
    glob = (448.0 * 6.0 / amax.max().clamp_min(1e-12)).reshape(1)             # dequant factor is 1 / glob
    scale = (amax / 6.0 * glob).to(torch.float8_e4m3fn)
    eff = (scale.float() / glob).clamp_min(1e-30)[..., None]
    lut = _lut(w.device)[:8]
    mag = (g.abs() / eff).clamp(max=6.0)
    code = (mag[..., None] - lut).abs().argmin(-1)                            # nearest representable magnitude
    code = code | ((g < 0) & (code > 0)).long() << 3
    code = code.view(n, k // 2, 2)
    packed = (code[..., 0] | (code[..., 1] << 4)).to(torch.uint8)
    return packed, scale, glob.float()


def dequantize(packed: torch.Tensor, scale: torch.Tensor, global_scale: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """-> [N, K] in ``dtype``."""
    n, kh = packed.shape
    lut = _lut(packed.device)
    p = packed.long()
    vals = torch.stack([lut[p & 0xF], lut[p >> 4]], -1).view(n, kh * 2 // GROUP, GROUP)
    s = scale.view(n, -1).float() / global_scale.float().reshape(())
    return (vals * s[..., None]).view(n, kh * 2).to(dtype)


def to_block64(packed: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """uint8 [N, K/64, 36]: per 64 values the four E4M3 group scales, then the 32 value bytes."""
    n, kh = packed.shape
    assert (kh * 2) % 64 == 0
    return torch.cat([scale.view(torch.uint8).view(n, -1, 4), packed.view(n, -1, 32)], -1).contiguous()


def from_block64(rec: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    n = rec.shape[0]
    return rec[..., 4:].reshape(n, -1).contiguous(), rec[..., :4].reshape(n, -1).contiguous().view(torch.float8_e4m3fn)
