"""Building blocks of the DeepSeek-V4 architecture that the MLA-shaped runtime does not use directly: YaRN rotary
tables with the complex-pair convention and de-rotation, the Hadamard-128 activation rotation, sliding-window and
compressed-block index tables, the learned KV compressor (prefill and incremental decode), the routing gate with
hash-table routing for the first layers, and the hyper-connection mixers (Sinkhorn-normalised combination weights).

Every function is the fp32 PyTorch statement of the math and runs on any device; ``hadamard128`` and the
hyper-connection mixers dispatch to sm_100a kernels for bf16 CUDA tensors (csrc/kernels/v4_ops.cu).

Reference behaviour: src/models/deepseek_v4/runtime.py - precompute_freqs_cis :898-926, apply_rotary_emb :929-942,
rotate_activation :945-951, window / compressed indices :954-1008, Compressor :1011-1109, Gate :1662-1731,
Block.hc_pre / hc_post :4369-4437; src/kernels/ops.py hc_split_sinkhorn :1224-1250.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------- rotary (YaRN)
def yarn_inv_freq(dim: int, base: float, factor: float = 1.0, original_seq_len: int = 0, beta_fast: float = 32.0,
                  beta_slow: float = 1.0) -> torch.Tensor:
    """Inverse frequencies [dim/2]; with ``original_seq_len > 0`` low frequencies are interpolated by ``factor`` with a
    linear ramp between the ``beta_fast`` and ``beta_slow`` rotation counts."""
    freqs = 1.0 / (base ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    if original_seq_len > 0:
        corr = lambda rot: dim * math.log(original_seq_len / (rot * 2 * math.pi)) / (2 * math.log(base))
        low, high = max(math.floor(corr(beta_fast)), 0), min(math.ceil(corr(beta_slow)), dim - 1)
        if low == high:
            high += 0.001
        smooth = 1 - ((torch.arange(dim // 2, dtype=torch.float32) - low) / (high - low)).clamp(0, 1)
        freqs = freqs / factor * (1 - smooth) + freqs * smooth
    return freqs


def rotary_table(dim: int, seqlen: int, base: float, factor: float = 1.0, original_seq_len: int = 0, beta_fast: float = 32.0,
                 beta_slow: float = 1.0) -> torch.Tensor:
    """complex64 [seqlen, dim/2]: e^{i t f}."""
    f = yarn_inv_freq(dim, base, factor, original_seq_len, beta_fast, beta_slow)
    ang = torch.outer(torch.arange(seqlen, dtype=torch.float32), f)
    return torch.polar(torch.ones_like(ang), ang)


def apply_rotary(x: torch.Tensor, table: torch.Tensor, inverse: bool = False) -> torch.Tensor:
    """Rotate consecutive pairs (x[2i], x[2i+1]) of the last dim by the table rows of each position; ``inverse`` applies
    the conjugate (used on the attention output).  x: [B, S, D] or [B, S, H, D]; table: [S, D/2]."""
    xc = torch.view_as_complex(x.float().unflatten(-1, (-1, 2)).contiguous())
    t = table.conj() if inverse else table
    t = t.view(1, x.size(1), xc.size(-1)) if xc.ndim == 3 else t.view(1, x.size(1), 1, xc.size(-1))
    return torch.view_as_real(xc * t).flatten(-2).to(x.dtype)


# ---------------------------------------------------------------------------------------------- Hadamard rotation
def hadamard128_ref(x: torch.Tensor) -> torch.Tensor:
    """Orthonormal Walsh-Hadamard transform over the last dim (128), fp32 butterflies."""
    assert x.shape[-1] == 128
    y = x.float().reshape(-1, 128)
    h = 1
    while h < 128:
        y = y.view(-1, 128 // (2 * h), 2, h)
        y = torch.stack([y[:, :, 0] + y[:, :, 1], y[:, :, 0] - y[:, :, 1]], 2).reshape(-1, 128)
        h *= 2
    return (y * 128 ** -0.5).reshape(x.shape).to(x.dtype)


def hadamard128(x: torch.Tensor) -> torch.Tensor:
    if x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous():
        from ..ops import v4 as v4ops
        return v4ops.hadamard128(x)
    return hadamard128_ref(x)


# ---------------------------------------------------------------------------------------------- index tables
def window_indices(window: int, seqlen: int, start_pos: int) -> torch.Tensor:
    """int64 [seqlen, window]: ring-buffer slots of the last ``window`` positions visible to each query (-1 = none).
    For a multi-token continuation the slots already overwritten by later tokens of the same chunk are masked."""
    if start_pos == 0:
        base = torch.arange(seqlen).unsqueeze(1)
        m = (base - window + 1).clamp(0) + torch.arange(min(seqlen, window))
        return torch.where(m > base, -1, m)
    rows = []
    for i in range(seqlen):
        cur = start_pos + i
        if cur >= window - 1:
            c = cur % window
            row = torch.cat([torch.arange(c + 1, window), torch.arange(0, c + 1)])
        else:
            row = F.pad(torch.arange(cur + 1), (0, window - cur - 1), value=-1)
        for j in range(i + 1, seqlen):
            row = torch.where(row == (start_pos + j) % window, torch.full_like(row, -1), row)
        rows.append(row)
    return torch.stack(rows)


def compressed_indices(ratio: int, seqlen: int, start_pos: int, offset: int) -> torch.Tensor:
    """int64 [seqlen, n]: compressed-block entries (shifted by ``offset`` into the cache) complete before each query."""
    if start_pos == 0:
        m = torch.arange(seqlen // ratio).repeat(seqlen, 1)
        mask = m >= torch.arange(1, seqlen + 1).unsqueeze(1) // ratio
        return torch.where(mask, -1, m + offset)
    rows = [torch.arange(0, (start_pos + i + 1) // ratio) + offset for i in range(seqlen)]
    n = max(r.numel() for r in rows)
    return torch.stack([F.pad(r, (0, n - r.numel()), value=-1) for r in rows])


# ---------------------------------------------------------------------------------------------- KV compressor
def _rms(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * g


class Compressor:
    """Learned pooling of ``ratio`` consecutive KV rows: soft-max weights from a gate projection plus a per-slot
    position bias ``ape``; ratio-4 layers pool over two overlapping windows (the previous block's first half of the
    channels and the current block's second half).  ``forward`` handles a prefill from position 0 and single-token
    continuation with running state, and returns the newly completed compressed rows (or None)."""

    def __init__(self, wkv: torch.Tensor, wgate: torch.Tensor, ape: torch.Tensor, norm: torch.Tensor, ratio: int, head_dim: int,
                 rope_dim: int, table: torch.Tensor, eps: float = 1e-6, max_batch: int = 1):
        self.wkv, self.wgate, self.ape, self.norm = wkv.float(), wgate.float(), ape.float(), norm.float()
        self.ratio, self.d, self.rd, self.table, self.eps = ratio, head_dim, rope_dim, table, eps
        self.overlap = ratio == 4
        coff = 1 + self.overlap
        dev = wkv.device
        self.kv_state = torch.zeros(max_batch, coff * ratio, coff * head_dim, device=dev)
        self.score_state = torch.full((max_batch, coff * ratio, coff * head_dim), float("-inf"), device=dev)

    def _overlap(self, t: torch.Tensor, value: float) -> torch.Tensor:
        b, s, r, _ = t.shape
        out = t.new_full((b, s, 2 * r, self.d), value)
        out[:, :, r:] = t[:, :, :, self.d:]
        out[:, 1:, :r] = t[:, :-1, :, :self.d]
        return out

    def forward(self, x: torch.Tensor, start_pos: int) -> torch.Tensor | None:
        b, s, _ = x.shape
        r, d = self.ratio, self.d
        xf = x.float()
        kv, score = xf @ self.wkv.t(), xf @ self.wgate.t()
        if start_pos == 0:
            rem = s % r
            cut = s - rem
            off = r if self.overlap else 0
            if self.overlap and cut >= r:
                self.kv_state[:b, :r] = kv[:, cut - r:cut]
                self.score_state[:b, :r] = score[:, cut - r:cut] + self.ape
            if rem > 0:
                self.kv_state[:b, off:off + rem] = kv[:, cut:]
                self.score_state[:b, off:off + rem] = score[:, cut:] + self.ape[:rem]
                kv, score = kv[:, :cut], score[:, :cut]
            if s < r:
                return None
            kv = kv.unflatten(1, (-1, r))
            score = score.unflatten(1, (-1, r)) + self.ape
            if self.overlap:
                kv, score = self._overlap(kv, 0.0), self._overlap(score, float("-inf"))
            out = (kv * score.softmax(2)).sum(2)
            pos = torch.arange(0, cut, r, device=x.device)
        else:
            assert s == 1
            slot = start_pos % r
            score = score + self.ape[slot]
            done = (start_pos + 1) % r == 0
            if self.overlap:
                self.kv_state[:b, r + slot] = kv[:, 0]
                self.score_state[:b, r + slot] = score[:, 0]
                if not done:
                    return None
                ks = torch.cat([self.kv_state[:b, :r, :d], self.kv_state[:b, r:, d:]], 1)
                ss = torch.cat([self.score_state[:b, :r, :d], self.score_state[:b, r:, d:]], 1)
                out = (ks * ss.softmax(1)).sum(1, keepdim=True)
                self.kv_state[:b, :r] = self.kv_state[:b, r:]
                self.score_state[:b, :r] = self.score_state[:b, r:]
            else:
                self.kv_state[:b, slot] = kv[:, 0]
                self.score_state[:b, slot] = score[:, 0]
                if not done:
                    return None
                out = (self.kv_state[:b] * self.score_state[:b].softmax(1)).sum(1, keepdim=True)
            pos = torch.tensor([start_pos + 1 - r], device=x.device)
        out = _rms(out, self.norm, self.eps)
        rot = apply_rotary(out[..., -self.rd:].contiguous(), self.table.to(x.device)[pos])
        return torch.cat([out[..., :-self.rd], rot], -1)


# ---------------------------------------------------------------------------------------------- routing gate
def gate_route(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor | None, topk: int, score_func: str,
               route_scale: float, tid2eid: torch.Tensor | None = None, input_ids: torch.Tensor | None = None
               ) -> tuple[torch.Tensor, torch.Tensor]:
    """(weights fp32 [T, k], indices int64 [T, k]).  The bias only steers the selection; hash layers take the experts of
    each token id from ``tid2eid`` [vocab, k] and still weight them by the scores."""
    scores = x.float() @ weight.float().t()
    scores = scores.softmax(-1) if score_func == "softmax" else scores.sigmoid() if score_func == "sigmoid" else \
        F.softplus(scores).sqrt()
    sel = scores if bias is None else scores + bias
    idx = tid2eid[input_ids].long() if tid2eid is not None else sel.topk(topk, -1)[1]
    w = scores.gather(1, idx)
    if score_func != "softmax":
        w = w / w.sum(-1, keepdim=True)
    return w * route_scale, idx


# ---------------------------------------------------------------------------------------------- hyper-connections
def hc_split_sinkhorn(mixes: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, hc: int = 4, iters: int = 20,
                      eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """mixes [..., (2 + hc) hc] -> pre [..., hc] (sigmoid), post [..., hc] (2 sigmoid), comb [..., hc, hc] made doubly
    stochastic by ``iters`` Sinkhorn normalisations."""
    flat = mixes.reshape(-1, (2 + hc) * hc).float()
    scale, base = scale.float(), base.float()
    pre = torch.sigmoid(flat[:, :hc] * scale[0] + base[:hc]) + eps
    post = 2 * torch.sigmoid(flat[:, hc:2 * hc] * scale[1] + base[hc:2 * hc])
    comb = (flat[:, 2 * hc:] * scale[2] + base[2 * hc:]).view(-1, hc, hc)
    comb = torch.softmax(comb, -1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(max(iters - 1, 0)):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    shape = mixes.shape[:-1]
    return pre.view(*shape, hc), post.view(*shape, hc), comb.view(*shape, hc, hc)


def hc_pre(x: torch.Tensor, fn: torch.Tensor, scale: torch.Tensor, base: torch.Tensor, norm_eps: float = 1e-6, iters: int = 20,
           eps: float = 1e-6) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """x [B, S, hc, D] streams -> (y [B, S, D] mixed input of the sub-layer, post [B, S, hc], comb [B, S, hc, hc])."""
    b, s, hc, d = x.shape
    flat = x.flatten(2).float()
    mixes = (flat @ fn.float().t()) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + norm_eps)
    if x.is_cuda and x.dtype == torch.bfloat16 and hc == 4:
        from ..ops import v4 as v4ops
        return v4ops.hc_split_pre(mixes, x, scale, base, iters, eps)
    pre, post, comb = hc_split_sinkhorn(mixes, scale, base, hc, iters, eps)
    return (pre.unsqueeze(-1) * x.float()).sum(2).to(x.dtype), post, comb


def hc_post(y: torch.Tensor, residual: torch.Tensor, post: torch.Tensor, comb: torch.Tensor) -> torch.Tensor:
    """Write the sub-layer output back: out[b, s, i] = post[i] y + sum_j comb[j, i] residual[j]."""
    if y.is_cuda and y.dtype == torch.bfloat16 and residual.size(2) == 4:
        from ..ops import v4 as v4ops
        return v4ops.hc_post(y, residual, post, comb)
    out = post.unsqueeze(-1) * y.float().unsqueeze(-2) + (comb.unsqueeze(-1) * residual.float().unsqueeze(-2)).sum(2)
    return out.to(y.dtype)
