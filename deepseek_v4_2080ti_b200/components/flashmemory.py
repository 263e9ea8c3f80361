"""FlashMemory: retrieval over compressed key chunks for contexts that do not fit (or need not stay) on the device.

Each scorer layer keeps one compressed key per chunk of the context (128 values, Hadamard-rotated; stored as E4M3 with
an fp32 scale, or as floats).  For a decode token the retriever projects the layer's hidden state to index queries,
scores every chunk, combines the scorer layers (max or mean), keeps the best chunks and maps them to KV row indices
behind the always-resident sliding window.  ``runtime/kv_swap.py`` keeps the KV rows of the other chunks in pinned host
memory.

The fp32 functions here are the oracle; ``FlashMemoryRetriever`` runs the sm_100a kernels of
``csrc/kernels/flashmemory.cu`` on CUDA tensors and the oracle elsewhere.

Reference behaviour: cpp_engine/include/flashmemory_ops.hpp:7-137 (score_layer, yarn_inv_freqs, ensemble, topk,
write_global_indices) and the plugin wiring in cpp_engine/engine/deepseek_v4_engine.cpp:75-340.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from ..models.v4_components import hadamard128_ref, yarn_inv_freq

D = 128


def yarn_inv_freqs(rope_dim: int, base: float, factor: float, original_seq_len: int, beta_fast: float = 32.0,
                   beta_slow: float = 1.0) -> torch.Tensor:
    """fp32 [rope_dim / 2] angular frequencies per rotated pair (YaRN mix of plain and interpolated frequencies)."""
    return yarn_inv_freq(rope_dim, base, factor, original_seq_len, beta_fast, beta_slow)


def compress_keys(keys: torch.Tensor) -> torch.Tensor:
    """fp32 [n, 128] -> uint8 [n, 132]: E4M3 bytes and the chunk's fp32 scale (amax / 448) in the last four bytes."""
    k = keys.float()
    scale = (k.abs().amax(-1, keepdim=True) / 448.0).clamp_min(1e-12)
    q = (k / scale).to(torch.float8_e4m3fn).view(torch.uint8)
    return torch.cat([q, scale.contiguous().view(torch.uint8).reshape(-1, 4)], 1).contiguous()


def decompress_keys(packed: torch.Tensor) -> torch.Tensor:
    scale = packed[:, D:].contiguous().view(torch.float32)
    return packed[:, :D].contiguous().view(torch.float8_e4m3fn).float() * scale


def _bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).float()


def build_query_ref(hidden, wq_a, wq_b, q_norm, inv_freqs, position: int, eps: float) -> torch.Tensor:
    """fp32 [heads, 128]: wq_a -> RMSNorm -> wq_b, bf16 rounding, RoPE on the last ``2 len(inv_freqs)`` dims (pairs
    (2i, 2i + 1)), Hadamard rotation."""
    h = hidden.float()
    ql = wq_a.float() @ h
    ql = ql * torch.rsqrt(ql.pow(2).mean() + eps) * q_norm.float()
    q = _bf16((wq_b.float() @ ql).view(-1, D))
    rope_dim = 2 * inv_freqs.numel()
    if rope_dim:
        ang = float(position) * inv_freqs.float()
        c, s = ang.cos(), ang.sin()
        tail = q[:, D - rope_dim:].reshape(-1, rope_dim // 2, 2)
        a, b = tail[..., 0], tail[..., 1]
        rot = torch.stack([_bf16(a * c - b * s), _bf16(a * s + b * c)], -1).reshape(-1, rope_dim)
        q = torch.cat([q[:, :D - rope_dim], rot], 1)
    return hadamard128_ref(q)


def score_layer_ref(hidden, wq_a, wq_b, q_norm, weights_proj, inv_freqs, keys, position: int, eps: float = 1e-6,
                    apply_sigmoid: bool = True) -> torch.Tensor:
    """fp32 [n_chunks]; ``keys`` are uint8 [n, 132] compressed chunks or fp32 [n, 128]."""
    q = build_query_ref(hidden, wq_a, wq_b, q_norm, inv_freqs, position, eps)
    heads = q.shape[0]
    fused_w = (weights_proj.float() @ hidden.float()) * (D ** -0.5) * (heads ** -0.5)
    k = decompress_keys(keys) if keys.dtype == torch.uint8 else keys.float()
    logit = (torch.relu(k @ q.t()) * fused_w).sum(-1)
    return torch.sigmoid(logit) if apply_sigmoid else logit


def ensemble_ref(layer_scores: torch.Tensor, use_max: bool = True) -> torch.Tensor:
    return layer_scores.amax(0) if use_max else layer_scores.mean(0)


def topk_ref(scores: torch.Tensor, keep: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Descending by score, ties to the lower chunk id; padded with -1 / -inf past the number of chunks."""
    n = scores.numel()
    order = torch.sort(scores.float(), descending=True, stable=True).indices[:keep]
    idx = torch.full((keep,), -1, dtype=torch.int32, device=scores.device)
    val = torch.full((keep,), float("-inf"), device=scores.device)
    idx[:min(keep, n)] = order.to(torch.int32)
    val[:min(keep, n)] = scores.float()[order]
    return idx, val


# ---------------------------------------------------------------------------------------------- retriever
@dataclass
class ScorerLayer:
    """Weights and chunk keys of one scorer layer.  ``keys`` is uint8 [capacity, 132] (compressed) or fp32
    [capacity, 128]; ``n_chunks`` of them are valid."""
    wq_a: torch.Tensor            # [q_lora, hidden]
    wq_b: torch.Tensor            # [heads * 128, q_lora]
    q_norm: torch.Tensor          # [q_lora]
    weights_proj: torch.Tensor    # [heads, hidden]
    keys: torch.Tensor
    n_chunks: int = 0

    def append(self, new_keys: torch.Tensor) -> None:
        """Add chunk keys (fp32 [m, 128]); compressed on the way in when the store is compressed."""
        m = new_keys.shape[0]
        if self.n_chunks + m > self.keys.shape[0]:
            raise RuntimeError("FlashMemory chunk store is full")
        rows = compress_keys(new_keys) if self.keys.dtype == torch.uint8 else new_keys.float()
        self.keys[self.n_chunks:self.n_chunks + m].copy_(rows.to(self.keys.device))
        self.n_chunks += m


class FlashMemoryRetriever:
    """Chunk selection for one sequence: ``select(hiddens, position)`` -> KV row indices of the kept chunks."""

    def __init__(self, layers: list[ScorerLayer], inv_freqs: torch.Tensor, chunk_tokens: int = 64, keep: int = 64,
                 window_offset: int = 0, use_max: bool = True, eps: float = 1e-6):
        assert layers and all(l.wq_b.shape[0] % D == 0 for l in layers)
        self.layers, self.chunk_tokens, self.keep, self.offset = layers, int(chunk_tokens), int(keep), int(window_offset)
        self.use_max, self.eps = bool(use_max), float(eps)
        dev = layers[0].keys.device
        self.device = dev
        self.inv_freqs = inv_freqs.float().to(dev).contiguous()
        self.capacity = min(l.keys.shape[0] for l in layers)
        self.cuda = dev.type == "cuda"
        if self.cuda:
            for l in layers:          # the kernels take bf16 matrices and fp32 vectors
                l.wq_a, l.wq_b = l.wq_a.to(dev, torch.bfloat16).contiguous(), l.wq_b.to(dev, torch.bfloat16).contiguous()
                l.weights_proj, l.q_norm = l.weights_proj.to(dev, torch.bfloat16).contiguous(), l.q_norm.to(dev, torch.float32).contiguous()
            heads = max(l.wq_b.shape[0] // D for l in layers)
            f32 = lambda *s: torch.empty(*s, dtype=torch.float32, device=dev)
            self._q, self._ql, self._fw = f32(heads * D), f32(max(l.wq_a.shape[0] for l in layers)), f32(heads)
            self._scores = f32(len(layers), self.capacity)
            self._ens = f32(self.capacity)
            self._idx = torch.empty(self.keep, dtype=torch.int32, device=dev)
            self._val = f32(self.keep)
            self._rows = torch.empty(self.keep, dtype=torch.int32, device=dev)

    @property
    def n_chunks(self) -> int:
        return min(l.n_chunks for l in self.layers)

    def scores(self, hiddens: list[torch.Tensor], position: int) -> torch.Tensor:
        """Ensembled chunk scores fp32 [n_chunks] for the decode token whose per-layer hidden states are ``hiddens``."""
        n = self.n_chunks
        if not self.cuda:
            per = torch.stack([score_layer_ref(h, l.wq_a, l.wq_b, l.q_norm, l.weights_proj, self.inv_freqs, l.keys[:n], position,
                                               self.eps) for h, l in zip(hiddens, self.layers)])
            return ensemble_ref(per, self.use_max)
        from ..ops import _lib
        L = _lib.lib()
        for i, (h, l) in enumerate(zip(hiddens, self.layers)):
            h32 = h.to(self.device, torch.float32).contiguous()
            heads, q_lora, hidden_dim = l.wq_b.shape[0] // D, l.wq_a.shape[0], l.wq_a.shape[1]
            k8 = l.keys if l.keys.dtype == torch.uint8 else None
            kf = l.keys if l.keys.dtype != torch.uint8 else None
            rc = L.b200_fm_score_layer(_lib.ptr(h32), _lib.ptr(l.wq_a), _lib.ptr(l.wq_b), _lib.ptr(l.q_norm),
                                       _lib.ptr(l.weights_proj), _lib.ptr(self.inv_freqs), _lib.ptr(k8), _lib.ptr(kf),
                                       _lib.ptr(self._q), _lib.ptr(self._ql), _lib.ptr(self._fw), _lib.ptr(self._scores[i]), n,
                                       heads, q_lora, hidden_dim, 2 * self.inv_freqs.numel(), ctypes.c_float(self.eps),
                                       ctypes.c_longlong(int(position)), 1, _lib.stream())
            _lib.check(rc, "fm_score_layer", 5)
        rc = L.b200_fm_ensemble(_lib.ptr(self._scores), len(self.layers), n, self.capacity, int(self.use_max),
                                _lib.ptr(self._ens), _lib.stream())
        _lib.check(rc, "fm_ensemble")
        return self._ens[:n]

    def select(self, hiddens: list[torch.Tensor], position: int) -> tuple[torch.Tensor, torch.Tensor]:
        """(chunk ids int32 [keep] by descending score, -1 = none; the same ids shifted by ``window_offset`` - the
        entries a layer's KV index list takes for its compressed region)."""
        s = self.scores(hiddens, position)
        if not self.cuda:
            idx, _ = topk_ref(s, self.keep)
            return idx, torch.where(idx < 0, idx, idx + self.offset)
        from ..ops import _lib
        L = _lib.lib()
        rc = L.b200_fm_topk(_lib.ptr(s), s.numel(), self.keep, _lib.ptr(self._idx), _lib.ptr(self._val), _lib.stream())
        _lib.check(rc, "fm_topk")
        rc = L.b200_fm_write_global_indices(_lib.ptr(self._idx), self.keep, self.offset, _lib.ptr(self._rows), _lib.stream())
        _lib.check(rc, "fm_write_global_indices")
        return self._idx, self._rows

    def token_rows(self, chunk_ids: torch.Tensor) -> torch.Tensor:
        """Token positions covered by the kept chunks, int32 [keep * chunk_tokens] (-1 for empty entries)."""
        base = chunk_ids.to(torch.int64)[:, None] * self.chunk_tokens + torch.arange(self.chunk_tokens, device=chunk_ids.device)
        return torch.where(chunk_ids[:, None] < 0, torch.full_like(base, -1), base).reshape(-1).to(torch.int32)
