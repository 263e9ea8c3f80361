"""The assembled DeepSeek-V4-style CPU runtime: window ring, compressed entries, indexer, hyper-connections, hash routing
and the MTP block must give the same logits token by token as in one pass over the prompt."""
import pytest
import torch

from deepseek_v4_2080ti_b200.models import v4_block_ref as v4
from deepseek_v4_2080ti_b200.models import v4_components as V


def _ids(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed))


def _stepwise(m, ids, n):
    m.reset()
    return torch.cat([m.forward(ids[:n])] + [m.forward(ids[i:i + 1]) for i in range(n, ids.numel())])


@pytest.mark.parametrize("kw", [{}, {"compress_ratios": (4, 4, 4), "n_hash_layers": 0, "score_func": "sigmoid"},
                                {"compress_ratios": (0, 16, 0), "score_func": "softmax", "n_hash_layers": 3, "window": 5},
                                {"hc_mult": 2, "n_heads": 6, "o_groups": 3, "swiglu_limit": 0.0, "mtp": False}])
def test_prefill_then_decode_matches_one_pass(kw):
    cfg = v4.V4Config(**kw)
    m = v4.V4BlockRef(cfg, v4.synth_weights(cfg, 0))
    ids = _ids(cfg, 45)
    full = m.forward(ids)
    assert full.shape == (45, cfg.vocab_size) and torch.isfinite(full).all()
    for n in (1, 3, 10, 23):                      # below / across the window, block boundaries and the index budget
        got = _stepwise(m, ids, n)
        assert torch.allclose(got, full, atol=5e-5, rtol=1e-4), (kw, n, (got - full).abs().max())


def test_indexer_only_matters_past_its_budget_and_window_ring_forgets():
    cfg = v4.V4Config(compress_ratios=(4, 4, 4))
    wide = v4.V4Config(compress_ratios=(4, 4, 4), index_topk=1000)
    w = v4.synth_weights(cfg, 2)
    a, b = v4.V4BlockRef(cfg, w).forward(_ids(cfg, 60, 3)), v4.V4BlockRef(wide, w).forward(_ids(cfg, 60, 3))
    exact = (cfg.index_topk + 1) * 4 - 1                  # up to index_topk complete blocks every entry is kept
    assert torch.allclose(a[:exact], b[:exact], atol=1e-5) and (a[exact:] - b[exact:]).abs().max() > 1e-4
    # a window-only model cannot see past its ring: changing the first token leaves late logits unchanged
    ring = v4.V4Config(compress_ratios=(0, 0, 0), n_hash_layers=0)
    m = v4.V4BlockRef(ring, v4.synth_weights(ring, 4))
    x = _ids(ring, 40, 5)
    y = x.clone(); y[0] = (y[0] + 1) % ring.vocab_size
    la, lb = m.forward(x), (m.reset(), m.forward(y))[1]
    reach = ring.n_layers * (ring.window - 1)             # receptive field of stacked windows
    assert (la[1] - lb[1]).abs().max() > 1e-5 and torch.allclose(la[reach + 1:], lb[reach + 1:], atol=1e-6)


def test_hash_layers_route_by_token_id_and_sink_takes_probability_mass():
    cfg = v4.V4Config()
    w = v4.synth_weights(cfg, 0)
    m = v4.V4BlockRef(cfg, w)
    layer = m.layers[0]
    x, ids = torch.randn(6, cfg.dim), _ids(cfg, 6, 9)
    _, idx = V.gate_route(x, w["layers.0.ffn.gate"], None, cfg.n_activated, cfg.score_func, cfg.route_scale,
                          w["layers.0.ffn.tid2eid"], ids)
    assert torch.equal(idx, w["layers.0.ffn.tid2eid"][ids]) and layer.hashed and not m.layers[1].hashed
    # attention over identical rows returns that row scaled by 1 - p(sink)
    q, kv = torch.randn(1, 2, 8), torch.randn(1, 8).repeat(3, 1)
    sink = torch.tensor([0.0, -30.0])
    o = v4.sparse_attention_ref(q, kv, sink, torch.tensor([[0, 1, 2, -1]]), 1.0)
    logit = (q[0] @ kv[0])
    keep = 3 * logit.exp() / (3 * logit.exp() + sink.exp())
    assert torch.allclose(o[0], keep[:, None] * kv[0], atol=1e-5) and keep[1] > 0.999


def test_mtp_draft_is_cache_consistent_and_speculative_loop_matches_greedy():
    cfg = v4.V4Config()
    m = v4.V4BlockRef(cfg, v4.synth_weights(cfg, 1))
    ids = _ids(cfg, 30, 7)
    m.forward(ids[:-1])
    full = m.draft(ids[1:])                               # MTP logits at every prompt position
    assert full.shape == (29, cfg.vocab_size)
    m.reset()
    m.forward(ids[:20]); parts = [m.draft(ids[1:21])]
    for i in range(20, 29):
        m.forward(ids[i:i + 1]); parts.append(m.draft(ids[i + 1:i + 2]))
    assert torch.allclose(torch.cat(parts), full, atol=5e-5, rtol=1e-4)
    toks, hits = m.generate_speculative(ids[:12], 8)
    assert toks == m.generate(ids[:12], 8) and 0 <= hits <= 7
    with pytest.raises(RuntimeError):
        m.forward(ids[:2])                                # a started sequence takes one token at a time


def test_snapshot_restore_resumes_a_shared_prefix_exactly():
    from deepseek_v4_2080ti_b200.runtime.prefix_cache import PrefixCache
    cfg = v4.V4Config()
    m = v4.V4BlockRef(cfg, v4.synth_weights(cfg, 0))
    ids = _ids(cfg, 40, 8)
    full = m.forward(ids)
    m.reset(); m.forward(ids[:24]); snap = m.snapshot()
    a = torch.cat([m.forward(ids[i:i + 1]) for i in range(24, 40)])
    m.reset(); m.forward(_ids(cfg, 30, 9))                    # unrelated traffic in between
    m.restore(snap)
    b = torch.cat([m.forward(ids[i:i + 1]) for i in range(24, 40)])
    assert torch.equal(a, b) and torch.allclose(a, full[24:], atol=5e-5, rtol=1e-4)
    # through the prefix cache: the state after 24 tokens is found again for a prompt that shares them
    cache = PrefixCache(interval=8, max_entries=4)
    toks = ids.tolist()
    assert cache.insert(toks, 24, [], snap, 1 << 10)
    other = toks[:24] + _ids(cfg, 6, 10).tolist()
    hit = cache.lookup(other)
    assert hit is not None and hit.tokens == 24
    m.restore(hit.snapshot)
    got = torch.cat([m.forward(torch.tensor([t])) for t in other[24:]])
    m.reset()
    assert torch.allclose(got, m.forward(torch.tensor(other))[24:], atol=5e-5, rtol=1e-4)
