"""Building blocks of the Qwen4-Exp (Qwen3.8-Flash-Next-style) family beyond what the hybrid runtime already has
(Gated DeltaNet, gated RMSNorm): interleaved 3-D rotary embedding, the low-rank gated hyper-connection mixer with its
stream injection, hashed n-gram embedding row ids, the soft-max top-k router, and the block-pooled sparse-attention
indexer (QSA).  fp32 PyTorch statements of the math, device-agnostic; the selected-token indices of ``qsa_select`` are
in the layout the sparse attention kernels take (int32, -1 = empty).

Reference behaviour: src/models/qwen4_exp/layers.py - MRoPE :288-326, GatedResidual :329-457, inject_into_streams
:460-491, NGramHasher :524-587, TopKRouter :590-606; src/models/qwen4_exp/attention.py QSAIndexer :461-594.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------------------------------------- MRoPE
def mrope_cos_sin(position_ids: torch.Tensor, rotary_dim: int, theta: float, sections: tuple[int, int, int],
                  dtype=torch.float32) -> tuple[torch.Tensor, torch.Tensor]:
    """position_ids [3, B, S] (text / height / width) or [B, S] -> cos, sin [B, S, rotary_dim].  The frequencies of
    the three axes are interleaved T H W T H W ...; the part beyond 3 * section length stays on the text axis."""
    if position_ids.ndim == 2:
        position_ids = position_ids[None].expand(3, -1, -1)
    inv = 1.0 / (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32, device=position_ids.device) / rotary_dim))
    freqs = position_ids[..., None].float() * inv                     # [3, B, S, rotary_dim / 2]
    out = freqs[0].clone()
    for axis, offset in ((1, 1), (2, 2)):
        idx = slice(offset, sections[axis] * 3, 3)
        out[..., idx] = freqs[axis][..., idx]
    emb = torch.cat([out, out], -1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def apply_rotary_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B, S, H, D]: rotate the first ``cos.shape[-1]`` dims, halves convention (x1, x2) -> (x1 c - x2 s, x2 c + x1 s)."""
    rd = cos.shape[-1]
    xr, rest = x[..., :rd].float(), x[..., rd:]
    x1, x2 = xr[..., :rd // 2], xr[..., rd // 2:]
    rot = torch.cat([-x2, x1], -1)
    out = xr * cos.unsqueeze(2).float() + rot * sin.unsqueeze(2).float()
    return torch.cat([out.to(x.dtype), rest], -1)


# ---------------------------------------------------------------------------------------------- hyper-connections
def _group_rms(x: torch.Tensor, gamma: torch.Tensor, group: int, eps: float) -> torch.Tensor:
    g = x.float().unflatten(-1, (-1, group))
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    return (g.flatten(-2) * gamma.float()).to(x.dtype)


def gated_residual(hyper: torch.Tensor, hc_norm: torch.Tensor, mix_down: torch.Tensor, mix_up: torch.Tensor,
                   block_inject: torch.Tensor | None, hc_count: int, hidden: int, eps: float = 1e-6):
    """hyper [..., hc_count * hidden] residual streams -> the block input: a gated mean of the (per-stream normalised)
    streams, gate = sigmoid(up(silu(down(x) / hc))).  With ``block_inject`` also returns the per-stream injection
    weights 2 sigmoid(inject(x) / hc) used to write the block output back."""
    normed = _group_rms(hyper, hc_norm, hidden, eps)
    down = F.silu(F.linear(normed.float(), mix_down.float()) / hc_count)
    w = torch.sigmoid(F.linear(down, mix_up.float())).unflatten(-1, (hc_count, hidden))
    mixed = (w * normed.float().unflatten(-1, (hc_count, hidden))).mean(-2).to(hyper.dtype)
    if block_inject is None:
        return mixed
    inject = 2 * torch.sigmoid(F.linear(normed.float(), block_inject.float()) / hc_count)
    return mixed, inject.to(hyper.dtype)


def inject_into_streams(block_output: torch.Tensor, hyper: torch.Tensor, inject: torch.Tensor) -> torch.Tensor:
    """hyper[..., g, :] += inject[..., g] * block_output for every stream g."""
    return hyper + (block_output.unsqueeze(-2) * inject.unsqueeze(-1)).flatten(-2)


# ---------------------------------------------------------------------------------------------- hashed n-grams
_MASK64 = (1 << 64) - 1
_GAMMA, _M1, _M2, _PRIME = 0x9E3779B97F4A7C15, 0xBF58476D1CE4E5B9, 0x94D049BB133111EB, 10007


def _splitmix64(v: int) -> int:
    v = (v + _GAMMA) & _MASK64
    v = ((v ^ (v >> 30)) * _M1) & _MASK64
    v = ((v ^ (v >> 27)) * _M2) & _MASK64
    return (v ^ (v >> 31)) & _MASK64


def ngram_multipliers(vocab: int, ngram_size: int, layer_index: int, seed: int) -> torch.Tensor:
    """Odd per-position hash multipliers derived from the seed (int64 [ngram_size])."""
    half = max(1, (((1 << 63) - 1) // max(vocab, 1)) // 2)
    base = seed + _PRIME * layer_index
    return torch.tensor([2 * (_splitmix64((base + _GAMMA * (i + 1)) & _MASK64) % half) + 1 for i in range(ngram_size)],
                        dtype=torch.long)


def _shift_right_within_document(tokens: torch.Tensor, shift: int, eos: int) -> torch.Tensor:
    if shift == 0:
        return tokens
    b, s = tokens.shape
    pos = torch.arange(s)
    eos_pos = torch.where(tokens == eos, pos, -1)
    prev_incl = torch.cummax(eos_pos, 1).values
    prev = torch.cat([eos_pos.new_full((b, 1), -1), prev_incl[:, :-1]], 1)
    in_seg = pos.unsqueeze(0) - (prev + 1)
    src = pos - shift
    shifted = tokens.gather(1, src.clamp_min(0).unsqueeze(0).expand(b, -1))
    ok = (in_seg >= shift) & (src.unsqueeze(0) >= 0)
    return torch.where(ok, shifted, tokens.new_full((), eos))


def ngram_row_ids(token_history: torch.Tensor, out_len: int, ngram_size: int, heads_per_ngram: int,
                  head_vocab_sizes: torch.Tensor, head_offsets: torch.Tensor, multipliers: torch.Tensor, eos: int) -> torch.Tensor:
    """token_history int64 [B, context + out_len] -> embedding-table rows [B, out_len, (ngram_size - 1) * heads].
    For every order n = 2..ngram_size the n most recent tokens (never crossing an end-of-document token) are mixed by
    XOR of per-position multiples and reduced modulo each head's (prime) table size."""
    t = token_history.to("cpu", torch.long)
    shifted = [_shift_right_within_document(t, s, eos) for s in range(ngram_size)]
    blocks = []
    for n in range(2, ngram_size + 1):
        lo = (n - 2) * heads_per_ngram
        mixed = shifted[0] * multipliers[0]
        for p in range(1, n):
            mixed = torch.bitwise_xor(mixed, shifted[p] * multipliers[p])
        sizes = head_vocab_sizes[lo:lo + heads_per_ngram].view(1, 1, -1)
        blocks.append(torch.remainder(mixed.unsqueeze(-1), sizes) + head_offsets[lo:lo + heads_per_ngram].view(1, 1, -1))
    return torch.cat(blocks, -1)[:, -out_len:]


# ---------------------------------------------------------------------------------------------- router
def topk_softmax_router(hidden: torch.Tensor, weight: torch.Tensor, top_k: int, norm_topk: bool = True):
    probs = F.softmax(F.linear(hidden.float(), weight.float()), -1)
    val, idx = probs.topk(top_k, -1)
    if norm_topk:
        val = val / val.sum(-1, keepdim=True)
    return val, idx


# ---------------------------------------------------------------------------------------------- QSA indexer
def qsa_select(q: torch.Tensor, raw_keys: torch.Tensor, k_gamma: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, past_len: int,
               budget: int, ratio: int, eps: float = 1e-6) -> torch.Tensor:
    """Token budget per query from mean-pooled key blocks.

    q [B, S, Hi, D] index queries (already normalised and rotated), raw_keys [B, kv_len, D] un-rotated index keys of
    the whole context, cos / sin [B, kv_len, D] rotary tables by absolute position.  Keys are averaged in groups of
    ``ratio``, normalised, rotated at the group's first position and scored by sum_h relu(q_h . k) / sqrt(D); the top
    ``budget / ratio`` complete blocks visible to a query expand to token ids, and the ragged tail after the last
    complete block is always kept.  Returns int32 [B, S, width], -1 = empty; width is kv_len on the dense path and
    min(budget // ratio, blocks) * ratio + ratio - 1 on the sparse one."""
    b, s, _, d = q.shape
    kv_len = raw_keys.shape[1]
    dev = q.device
    visible = past_len + torch.arange(s, device=dev) + 1
    if kv_len <= budget or kv_len // ratio == 0:
        ids = torch.arange(kv_len, device=dev).view(1, 1, -1).expand(b, s, -1)
        ids = ids.masked_fill(ids >= visible.view(1, -1, 1), -1)
        return ids.to(torch.int32)
    nblk = kv_len // ratio
    block_tokens = torch.arange(nblk * ratio, device=dev).view(nblk, ratio)
    pooled = raw_keys[:, :nblk * ratio].reshape(b, nblk, ratio, d).float().mean(2)
    pooled = pooled * torch.rsqrt(pooled.pow(2).mean(-1, keepdim=True) + eps) * k_gamma.float()
    starts = block_tokens[:, 0]
    bk = apply_rotary_half(pooled.unsqueeze(2), cos[:, starts], sin[:, starts]).squeeze(2)
    scores = torch.relu(torch.einsum("bqhd,bkd->bqhk", q.float(), bk.float())).sum(2) / math.sqrt(d)
    blocks_visible = visible // ratio
    ok = torch.arange(nblk, device=dev).view(1, -1) < blocks_visible.view(-1, 1)
    scores = scores.masked_fill(~ok.unsqueeze(0), float("-inf"))
    topk = min(budget // ratio, nblk)
    # relu makes exact zero scores common; ties go to the lower block id so that the choice does not depend on how many
    # later blocks exist
    sel = torch.sort(scores, dim=-1, descending=True, stable=True).indices[..., :topk]
    sel_ok = torch.gather(ok.unsqueeze(0).expand(b, -1, -1), 2, sel)
    toks = block_tokens[sel].reshape(b, s, -1).masked_fill(~sel_ok.unsqueeze(-1).expand(-1, -1, -1, ratio).reshape(b, s, -1), -1)
    tail = (blocks_visible * ratio).view(1, s, 1) + torch.arange(ratio - 1, device=dev).view(1, 1, -1)
    tail = tail.expand(b, -1, -1).masked_fill(~(tail < visible.view(1, s, 1)).expand(b, -1, -1), -1)
    # Every slot is kept: topk * ratio block tokens then ratio - 1 tail slots.  (Cutting the row to kv_len, as the
    # reference does when budget < kv_len < budget + ratio - 1, drops tail tokens of the early queries of a prefill
    # chunk and makes the result depend on where the prompt was split.)
    return torch.cat([toks, tail], -1).to(torch.int32)
