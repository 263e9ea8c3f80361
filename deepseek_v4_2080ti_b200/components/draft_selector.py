"""Choosing one token per position of a drafted block from per-position candidate lists with a first-order chain score.

A block drafter that predicts all positions at once (a diffusion-style block) gives, per position p, ``K`` candidate
tokens with unary scores; a low-rank selector links neighbours:

    edge_p(prev, tok) = unary[p, tok] + sum_r predecessor[prev, r] * projected[p, r] * successor[tok, r]

with ``projected = hidden @ selector_projection^T`` [rows, rank].  ``greedy_path`` takes the best candidate at each
position given its own previous pick (starting from the anchor token); ``viterbi_path`` returns the exact maximum of
the summed edge scores over all K^rows paths in rows * K^2 edge evaluations.  Ties go to the smaller token id.  Both
are plain tensor code and run on whatever device the inputs live on (rows and K are at most a few dozen).

Reference behaviour: cpp_engine/backends/cuda/kernels/qwen_dflash2_ops.cu:690-860 (selector_path_projected_kernel,
selector_path_viterbi_kernel) and the selector projection :664-688.
"""
from __future__ import annotations

import torch


def project(hidden: torch.Tensor, selector_projection: torch.Tensor) -> torch.Tensor:
    """hidden [rows, H], selector_projection [rank, H] -> fp32 [rows, rank]."""
    return hidden.float() @ selector_projection.float().t()


def _edges(prev_tokens: torch.Tensor, cand: torch.Tensor, unary: torch.Tensor, proj: torch.Tensor, predecessor: torch.Tensor,
           successor: torch.Tensor) -> torch.Tensor:
    """Scores [P, K] of moving from each of ``prev_tokens`` [P] to each of ``cand`` [K] at a position with ``proj`` [rank]."""
    left = predecessor[prev_tokens].float() * proj                                     # [P, rank]
    return unary.float()[None, :] + left @ successor[cand].float().t()


def _argmax_low_token(scores: torch.Tensor, tokens: torch.Tensor) -> int:
    """Index of the best score; among equal scores the smallest token id."""
    best = scores == scores.max()
    return int(torch.where(best, tokens, torch.full_like(tokens, torch.iinfo(tokens.dtype).max)).argmin())


def greedy_path(projected: torch.Tensor, candidates: torch.Tensor, unary: torch.Tensor, predecessor: torch.Tensor,
                successor: torch.Tensor, anchor_token: int) -> tuple[list[int], float]:
    """candidates int [rows, K], unary [rows, K] -> (tokens [rows], summed score)."""
    prev, out, total = int(anchor_token), [], 0.0
    for p in range(candidates.shape[0]):
        cand = candidates[p].long()
        s = _edges(torch.tensor([prev], device=cand.device), cand, unary[p], projected[p], predecessor, successor)[0]
        k = _argmax_low_token(s, cand)
        total += float(s[k])
        prev = int(cand[k])
        out.append(prev)
    return out, total


def viterbi_path(projected: torch.Tensor, candidates: torch.Tensor, unary: torch.Tensor, predecessor: torch.Tensor,
                 successor: torch.Tensor, anchor_token: int) -> tuple[list[int], float]:
    """Exact best path.  With K = 1 it is the greedy path."""
    rows, K = candidates.shape
    dev = candidates.device
    cand = candidates.long()
    dp = _edges(torch.tensor([int(anchor_token)], device=dev), cand[0], unary[0], projected[0], predecessor, successor)[0]
    back = torch.zeros(rows, K, dtype=torch.long, device=dev)
    for p in range(1, rows):
        e = dp[:, None] + _edges(cand[p - 1], cand[p], unary[p], projected[p], predecessor, successor)     # [prev K, K]
        best = e.max(0).values
        # among equally good predecessors keep the smaller token id, as the greedy rule would
        tie = torch.where(e == best[None, :], cand[p - 1][:, None].expand(K, K), torch.full((K, K), torch.iinfo(torch.long).max, device=dev))
        back[p] = tie.argmin(0)
        dp = best
    k = _argmax_low_token(dp, cand[-1])
    total, path = float(dp[k]), []
    for p in range(rows - 1, -1, -1):
        path.append(int(cand[p, k]))
        k = int(back[p, k])
    return path[::-1], total


def path_score(tokens: list[int], projected: torch.Tensor, candidates: torch.Tensor, unary: torch.Tensor,
               predecessor: torch.Tensor, successor: torch.Tensor, anchor_token: int) -> float:
    """Summed edge score of a given path (each token must be among its position's candidates)."""
    prev, total = int(anchor_token), 0.0
    for p, t in enumerate(tokens):
        k = int((candidates[p] == t).nonzero()[0])
        total += float(_edges(torch.tensor([prev], device=candidates.device), candidates[p, k:k + 1].long(), unary[p, k:k + 1],
                              projected[p], predecessor, successor)[0, 0])
        prev = int(t)
    return total


# ---------------------------------------------------------------------------------------------- block-drafter pieces
def grouped_dynamic_conv(hidden: torch.Tensor, dynamic: torch.Tensor, base: torch.Tensor, group_size: int) -> torch.Tensor:
    """Causal depthwise convolution over the rows of a drafted block whose taps are a learned base kernel plus a
    per-row correction shared by groups of channels:

        out[r, c] = sum_t hidden[r - t, c] * (base[t, c] + dynamic[r, t * G + c // group_size]),   rows before 0 are zero

    hidden [rows, H], base [K, H], dynamic [rows, K * G] with G = H / group_size (the row's own projection of its hidden
    state).  fp32 result.  Reference behaviour: qwen_dflash2_ops.cu:81-117 (grouped_dynamic_conv_kernel)."""
    rows, h = hidden.shape
    k = base.shape[0]
    g = h // group_size
    assert h % group_size == 0 and dynamic.shape == (rows, k * g)
    x = hidden.float()
    taps = base.float()[None, :, :] + dynamic.float().view(rows, k, g).repeat_interleave(group_size, dim=2)      # [rows, K, H]
    out = torch.zeros(rows, h, dtype=torch.float32, device=hidden.device)
    for t in range(min(k, rows)):
        out[t:] += x[:rows - t] * taps[t:, t]
    return out


def sharded_topk(logit_shards: list[torch.Tensor], k: int) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-position candidates from a vocabulary-sharded head: every shard [rows, V_s] contributes its own top ``k``,
    the winners are merged.  Returns (token ids int64 [rows, k], logits [rows, k]) sorted by descending logit, equal
    logits by ascending token id - the ``candidates`` / ``unary`` inputs of the selector.
    Reference behaviour: the local top-k + gather of qwen_dflash2.cpp:1100-1170."""
    ids, vals, off = [], [], 0
    for sh in logit_shards:
        kk = min(k, sh.shape[1])
        i = torch.argsort(sh.float(), dim=-1, descending=True, stable=True)[:, :kk]       # ties at the cut: lower id stays
        v = sh.float().gather(-1, i)
        ids.append(i + off)
        vals.append(v)
        off += sh.shape[1]
    ids, vals = torch.cat(ids, -1), torch.cat(vals, -1)
    order = torch.argsort(ids, dim=-1, stable=True)                          # ascending id first, then a stable sort by value
    ids, vals = ids.gather(-1, order), vals.gather(-1, order)
    order = torch.argsort(vals, dim=-1, descending=True, stable=True)[:, :k]
    return ids.gather(-1, order), vals.gather(-1, order)
