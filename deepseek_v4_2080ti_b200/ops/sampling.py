"""Device-side token sampling (csrc/kernels/sampling.cu): penalties, temperature, top-k, top-p, min-p.

``sample`` works on this rank's vocabulary shard of the logits; with a tensor-parallel communicator the per-rank
candidates are gathered and the draw is made on the merged list, identically on every rank (same uniforms)."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

import torch

from . import _lib, mla

MAX_CANDIDATES = 1024


@dataclass
class DeviceSampling:
    temperature: float = 1.0
    top_k: int = 0                 # 0 = off (the 1024 most likely tokens are the candidate set)
    top_p: float = 1.0
    min_p: float = 0.0
    repetition_penalty: float = 1.0
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0

    @staticmethod
    def from_params(sp) -> "DeviceSampling | None":
        """From an API ``SamplingParams``-like object; None when the request is greedy."""
        if sp is None or not getattr(sp, "temperature", 0.0):
            return None
        return DeviceSampling(float(sp.temperature), int(getattr(sp, "top_k", 0) or 0), float(getattr(sp, "top_p", None) or 1.0),
                              float(getattr(sp, "min_p", None) or 0.0), float(getattr(sp, "repetition_penalty", 1.0) or 1.0),
                              float(getattr(sp, "presence_penalty", 0.0) or 0.0),
                              float(getattr(sp, "frequency_penalty", 0.0) or 0.0))

    @property
    def has_penalties(self) -> bool:
        return self.repetition_penalty != 1.0 or self.presence_penalty != 0.0 or self.frequency_penalty != 0.0


def apply_penalties(logits: torch.Tensor, counts: torch.Tensor, s: DeviceSampling) -> torch.Tensor:
    """In place on fp32 ``logits`` [B, n]; ``counts`` int32 [B, n] occurrences of each id in the sequence so far."""
    b, n = logits.shape
    rc = _lib.lib().b200_apply_penalties(_lib.ptr(logits), logits.stride(0), n, b, _lib.ptr(counts),
                                         ctypes.c_float(s.repetition_penalty), ctypes.c_float(s.presence_penalty),
                                         ctypes.c_float(s.frequency_penalty), _lib.stream())
    _lib.check(rc, "apply_penalties")
    return logits


def _draw(vals: torch.Tensor, idx: torch.Tensor, s: DeviceSampling, u: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    b, k = idx.shape
    pos = torch.empty(b, dtype=torch.int32, device=vals.device)
    prob = torch.empty(b, dtype=torch.float32, device=vals.device)
    rc = _lib.lib().b200_sample_candidates(_lib.ptr(vals), vals.stride(0), _lib.ptr(idx), k, b, ctypes.c_float(s.temperature),
                                           ctypes.c_float(s.top_p), ctypes.c_float(s.min_p), _lib.ptr(u), _lib.ptr(pos),
                                           _lib.ptr(prob), _lib.stream())
    _lib.check(rc, "sample_candidates")
    return pos, prob


def sample(logits: torch.Tensor, s: DeviceSampling, u: torch.Tensor, index_offset: int = 0, comm=None,
           counts: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``logits`` [B, n_local] -> token ids int32 [B].  ``u``: fp32 [B] uniforms in [0, 1) (identical on every
    rank).  ``index_offset``: first vocabulary id of this rank's shard."""
    assert logits.dtype == torch.float32 and logits.dim() == 2
    b, n = logits.shape
    if counts is not None and s.has_penalties:
        logits = apply_penalties(logits.clone(), counts, s)
    k = min(s.top_k if s.top_k > 0 else MAX_CANDIDATES, MAX_CANDIDATES, n)
    nv = torch.full((b,), n, dtype=torch.int32, device=logits.device)
    idx = mla.topk_rows(logits, nv, k)
    world = getattr(comm, "world", 1) if comm is not None else 1
    if world == 1:
        pos, _ = _draw(logits, idx, s, u)
        return (pos + index_offset).to(torch.int32)
    # merge the shards' candidates: values and global ids
    safe = idx.clamp_min(0).long()
    vals = torch.where(idx >= 0, logits.gather(1, safe), torch.full_like(logits[:, :1], float("-inf")).expand(b, k))
    gids = torch.where(idx >= 0, idx + index_offset, idx)
    all_vals = comm.all_gather(vals.contiguous()).permute(1, 0, 2).reshape(b, world * k).contiguous()
    all_ids = comm.all_gather(gids.contiguous()).permute(1, 0, 2).reshape(b, world * k).contiguous()
    nv2 = torch.full((b,), world * k, dtype=torch.int32, device=logits.device)
    idx2 = mla.topk_rows(all_vals, nv2, k)
    pos, _ = _draw(all_vals, idx2, s, u)
    return all_ids.gather(1, pos.long()[:, None])[:, 0].to(torch.int32)


def sample_ref(logits: torch.Tensor, s: DeviceSampling, u: torch.Tensor) -> torch.Tensor:
    """fp32 PyTorch restatement (same candidate cap, same tie order, same inverse-CDF draw)."""
    b, n = logits.shape
    k = min(s.top_k if s.top_k > 0 else MAX_CANDIDATES, MAX_CANDIDATES, n)
    out = []
    for r in range(b):
        v, i = torch.sort(logits[r].double(), descending=True, stable=True)
        v, i = v[:k], i[:k]
        p = torch.softmax(v / s.temperature, 0)
        keep, cum = 0, 0.0
        for j in range(k):
            if j > 0 and (p[j] < s.min_p * p[0] or cum >= s.top_p):
                break
            cum += float(p[j])
            keep += 1
        target, acc, pick = float(u[r]) * cum, 0.0, 0
        for j in range(keep):
            acc += float(p[j])
            pick = j
            if acc > target:
                break
        out.append(int(i[pick]))
    return torch.tensor(out, dtype=torch.int32)
