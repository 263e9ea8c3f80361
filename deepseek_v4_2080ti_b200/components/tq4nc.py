"""TQ4NC: 4-bit KV-cache quantiser with a non-uniform codebook (prototype).

Each vector is rotated by an orthonormal Hadamard transform (spreads outliers), scaled by its RMS, and every component
is mapped to the nearest of 16 levels placed at the quantiles of a standard normal (what the rotated, normalised
components follow); two codes share a byte.  Storage per vector of dim D: D/2 bytes + one fp16 scale.
Reference behaviour: src/kernels/tq4nc_quantizer.py (prototype only, not wired into a serving path there either)."""
from __future__ import annotations

import torch


def _hadamard(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1]
    assert d & (d - 1) == 0, "power-of-two width"
    y = x.float().reshape(-1, d)
    h = 1
    while h < d:
        y = y.view(-1, d // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], 2).reshape(-1, d)
        h *= 2
    return (y * d ** -0.5).reshape(x.shape)


_CB: torch.Tensor | None = None


def codebook(device="cpu") -> torch.Tensor:
    """16 Lloyd-Max levels of a standard normal: start from equal-probability bins, then alternate bin edges at the
    level midpoints and levels at the conditional means (closed form through the normal pdf / cdf)."""
    global _CB
    if _CB is None:
        n = torch.distributions.Normal(torch.tensor(0.0, dtype=torch.float64), torch.tensor(1.0, dtype=torch.float64))
        pdf = lambda z: torch.exp(-0.5 * z * z) / (2 * torch.pi) ** 0.5
        inner = n.icdf(torch.linspace(0, 1, 17, dtype=torch.float64)[1:-1])
        big = torch.tensor([40.0], dtype=torch.float64)
        for _ in range(200):
            edges = torch.cat([-big, inner, big])
            lo, hi = edges[:-1], edges[1:]
            levels = (pdf(lo) - pdf(hi)) / (n.cdf(hi) - n.cdf(lo))
            inner = 0.5 * (levels[1:] + levels[:-1])
        _CB = levels.float()
    return _CB.to(device)


def quantize(x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """x [..., D] -> (codes uint8 [..., D/2], scale fp16 [...])."""
    r = _hadamard(x)
    scale = r.pow(2).mean(-1, keepdim=True).sqrt().clamp_min(1e-12)
    cb = codebook(x.device)
    idx = ((r / scale).unsqueeze(-1) - cb).abs().argmin(-1).to(torch.uint8)
    return idx[..., 0::2] | (idx[..., 1::2] << 4), scale.squeeze(-1).half()


def dequantize(codes: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    cb = codebook(codes.device)
    idx = torch.stack([codes & 0xF, codes >> 4], -1).flatten(-2).long()
    return _hadamard(cb[idx] * scale.float().unsqueeze(-1))          # the transform is its own inverse
