"""First-order selector over a drafted block: greedy chain and exact (Viterbi) path."""
import itertools

import torch

from deepseek_v4_2080ti_b200.components import draft_selector as sel


def _problem(rows, K, vocab=40, rank=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    cand = torch.stack([torch.randperm(vocab, generator=g)[:K] for _ in range(rows)])
    unary = torch.randn(rows, K, generator=g)
    hidden, projm = torch.randn(rows, 16, generator=g), torch.randn(rank, 16, generator=g) * 0.4
    pred, succ = torch.randn(vocab, rank, generator=g), torch.randn(vocab, rank, generator=g)
    return sel.project(hidden, projm), cand, unary, pred, succ


def test_viterbi_is_the_brute_force_maximum_and_never_below_greedy():
    worse = 0
    for seed in range(6):
        proj, cand, unary, pred, succ = _problem(4, 3, seed=seed)
        best = max((sel.path_score([int(cand[p, k]) for p, k in enumerate(ks)], proj, cand, unary, pred, succ, 7), ks)
                   for ks in itertools.product(range(3), repeat=4))
        path, total = sel.viterbi_path(proj, cand, unary, pred, succ, 7)
        assert abs(total - best[0]) < 1e-4 and path == [int(cand[p, k]) for p, k in enumerate(best[1])]
        assert abs(sel.path_score(path, proj, cand, unary, pred, succ, 7) - total) < 1e-4
        gpath, gtotal = sel.greedy_path(proj, cand, unary, pred, succ, 7)
        assert gtotal <= total + 1e-5
        worse += int(gtotal < total - 1e-4)
        assert abs(sel.path_score(gpath, proj, cand, unary, pred, succ, 7) - gtotal) < 1e-4
    assert worse > 0                                        # the chain term makes greedy miss the optimum sometimes


def test_single_candidate_and_long_block():
    proj, cand, unary, pred, succ = _problem(8, 1, seed=3)
    (vp, vs), (gp, gs) = sel.viterbi_path(proj, cand, unary, pred, succ, 0), sel.greedy_path(proj, cand, unary, pred, succ, 0)
    assert vp == gp and abs(vs - gs) < 1e-5
    proj, cand, unary, pred, succ = _problem(8, 16, vocab=300, rank=32, seed=4)
    path, total = sel.viterbi_path(proj, cand, unary, pred, succ, 5)
    assert len(path) == 8 and all(path[p] in cand[p].tolist() for p in range(8))
    assert total >= sel.greedy_path(proj, cand, unary, pred, succ, 5)[1] - 1e-5


def test_ties_go_to_the_smaller_token_and_the_anchor_matters():
    rows, K, rank = 3, 3, 2
    cand = torch.tensor([[9, 4, 6], [8, 2, 5], [3, 7, 1]])
    zeros = torch.zeros(rows, K)
    pred = succ = torch.zeros(12, rank)
    proj = torch.ones(rows, rank)
    assert sel.greedy_path(proj, cand, zeros, pred, succ, 0)[0] == [4, 2, 1]
    assert sel.viterbi_path(proj, cand, zeros, pred, succ, 0)[0] == [4, 2, 1]
    # a chain term that rewards prev == 10 -> token 6 only: the anchor decides the first pick
    pred = torch.zeros(12, rank); succ = torch.zeros(12, rank)
    pred[10, 0] = 1.0; succ[6, 0] = 2.0
    assert sel.greedy_path(proj, cand, zeros, pred, succ, 10)[0][0] == 6
    assert sel.viterbi_path(proj, cand, zeros, pred, succ, 11)[0][0] == 4
