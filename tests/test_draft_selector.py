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


def test_grouped_dynamic_conv_matches_the_scalar_definition():
    g = torch.Generator().manual_seed(0)
    rows, h, k, gs = 8, 12, 3, 4
    hidden, base, dyn = torch.randn(rows, h, generator=g), torch.randn(k, h, generator=g), torch.randn(rows, k * (h // gs), generator=g)
    want = torch.zeros(rows, h)
    for r in range(rows):
        for c in range(h):
            for t in range(k):
                if r - t >= 0:
                    want[r, c] += hidden[r - t, c] * (base[t, c] + dyn[r, t * (h // gs) + c // gs])
    got = sel.grouped_dynamic_conv(hidden, dyn, base, gs)
    assert torch.allclose(got, want, atol=1e-5)
    # causal: a later row does not change earlier outputs; with a zero correction it is a plain depthwise convolution
    h2 = hidden.clone(); h2[5] += 1.0
    assert torch.equal(sel.grouped_dynamic_conv(h2, dyn, base, gs)[:5], got[:5])
    plain = sel.grouped_dynamic_conv(hidden, torch.zeros_like(dyn), base, gs)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(hidden.t()[None], (k - 1, 0)), base.flip(0).t()[:, None, :], groups=h)[0].t()
    assert torch.allclose(plain, ref, atol=1e-5)


def test_sharded_topk_equals_the_top_k_of_the_whole_vocabulary():
    g = torch.Generator().manual_seed(1)
    logits = torch.randn(5, 64, generator=g)
    logits[0, 10] = logits[0, 50] = 9.0                      # a tie across shards goes to the smaller id
    ids, vals = sel.sharded_topk(list(logits.split(16, -1)), 4)
    v, i = logits.topk(4, -1)
    assert torch.allclose(vals, v) and torch.equal(ids[1:], i[1:])
    assert ids[0, :2].tolist() == [10, 50]
    one, _ = sel.sharded_topk([logits], 4)
    assert torch.equal(one[1:], i[1:])
    # feeding the selector: with no chain term the path is the per-position arg-max
    proj, pred, succ = torch.zeros(5, 2), torch.zeros(64, 2), torch.zeros(64, 2)
    assert sel.viterbi_path(proj, ids, vals, pred, succ, 0)[0] == [int(ids[p, 0]) for p in range(5)]
