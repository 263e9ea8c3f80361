"""The assembled Qwen4-Exp-style CPU runtime: caches must reproduce the uncached forward pass, however the prompt is split."""
import pytest
import torch

from deepseek_v4_2080ti_b200.models import qwen4_exp_ref as q4


def _ids(cfg, n, seed=1):
    return torch.randint(1, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed))


def _chunked(m, ids, cuts):
    m.reset()
    out, prev = [], 0
    for c in list(cuts) + [ids.numel()]:
        out.append(m.forward(ids[prev:c]))
        prev = c
    return torch.cat(out)


@pytest.mark.parametrize("kw", [{}, {"ple_layers": ()}, {"layer_types": ["full"] * 4}, {"layer_types": ["linear"] * 4},
                                {"ple_layers": (0, 2), "ngram_size": 2, "ngram_head_vocab": (31, 37), "ple_conv_kernel": 3}])
def test_cached_forward_matches_one_pass(kw):
    cfg = q4.Qwen4ExpConfig(**kw)
    m = q4.Qwen4ExpRef(cfg, q4.synth_weights(cfg, 0), 128)
    ids = _ids(cfg, 45)
    full = m.forward(ids)
    assert full.shape == (45, cfg.vocab_size) and torch.isfinite(full).all()
    for cuts in ([17, 18, 19, 33], [1, 2, 3], list(range(30, 45))):          # 17..19 straddle budget .. budget + ratio - 1
        got = _chunked(m, ids, cuts)
        assert torch.allclose(got, full, atol=2e-5, rtol=1e-4), (kw, cuts, (got - full).abs().max())


def test_sparse_selection_changes_the_output_only_past_the_budget():
    cfg = q4.Qwen4ExpConfig()
    dense = q4.Qwen4ExpConfig(indexer_budget=4096)
    w = q4.synth_weights(cfg, 3)
    ms, md = q4.Qwen4ExpRef(cfg, w, 128), q4.Qwen4ExpRef(dense, w, 128)
    ids = _ids(cfg, 60, seed=5)
    a, b = ms.forward(ids), md.forward(ids)
    # a query sees everything while its complete blocks number at most budget / ratio: positions 0 .. budget + ratio - 2
    exact = cfg.indexer_budget + cfg.indexer_compress_ratio - 1
    assert torch.allclose(a[:exact], b[:exact], atol=2e-5)
    assert (a[exact:] - b[exact:]).abs().max() > 1e-4


def test_generate_is_deterministic_and_history_feeds_the_ngram_tables():
    cfg = q4.Qwen4ExpConfig()
    m = q4.Qwen4ExpRef(cfg, q4.synth_weights(cfg, 0), 128)
    prompt = _ids(cfg, 20)
    a = m.generate(prompt, 6, chunk=7)
    assert a == m.generate(prompt, 6, chunk=64) and len(a) == 6
    # the n-gram injection reads the token history across calls: the same token after different prefixes differs
    m.reset(); m.forward(torch.tensor([5, 6])); x = m.forward(torch.tensor([9]))
    m.reset(); m.forward(torch.tensor([7, 8])); y = m.forward(torch.tensor([9]))
    assert (x - y).abs().max() > 1e-6
    with pytest.raises(RuntimeError):
        q4.Qwen4ExpRef(cfg, q4.synth_weights(cfg, 0), 8).forward(_ids(cfg, 9))


def test_prefix_cache_resumes_recurrent_and_sparse_layers_exactly():
    from deepseek_v4_2080ti_b200.runtime.prefix_cache import PrefixCache
    cfg = q4.Qwen4ExpConfig()
    m = q4.Qwen4ExpRef(cfg, q4.synth_weights(cfg, 0), 160)
    cache = PrefixCache(interval=16, max_entries=8)
    shared = _ids(cfg, 50, seed=11)
    a = torch.cat([shared, _ids(cfg, 9, seed=12)])
    b = torch.cat([shared, _ids(cfg, 13, seed=13)])
    la, reused = m.prefill_cached(a, cache)
    assert reused == 0 and len(cache) == 3                                   # snapshots after 16, 32 and 48 tokens
    m.reset(); want_a = m.forward(a)[-1]
    assert torch.allclose(la, want_a, atol=2e-5)
    lb, reused = m.prefill_cached(b, cache)
    assert reused == 48 and cache.stats.hits == 1                            # longest shared boundary
    m.reset(); want_b = m.forward(b)[-1]
    assert torch.allclose(lb, want_b, atol=2e-5)
    # the same prompt again stops one boundary short of its end, so logits are still computed
    la2, reused = m.prefill_cached(a, cache)
    assert reused == 48 and torch.allclose(la2, want_a, atol=2e-5)


@pytest.mark.parametrize("kw,world", [({}, 2), ({"linear_k_heads": 2, "linear_v_heads": 4, "num_heads": 8, "num_kv_heads": 4}, 2),
                                      ({"linear_k_heads": 2, "linear_v_heads": 8, "num_heads": 8, "num_kv_heads": 4}, 4)])
def test_tensor_parallel_shards_reproduce_the_unsharded_model(kw, world):
    cfg = q4.Qwen4ExpConfig(**kw)
    w = q4.synth_weights(cfg, 0)
    ids = _ids(cfg, 40)
    full = q4.Qwen4ExpRef(cfg, w, 128).forward(ids)
    tp = q4.Qwen4ExpTP(cfg, w, world, 128)
    got = torch.cat([tp.forward(ids[:25]), tp.forward(ids[25:])])            # prefill, then a continuation on the caches
    assert torch.allclose(got, full, atol=2e-5, rtol=1e-4)
    # what a rank holds: its experts only, a slice of the heads, every replicated tensor whole
    rcfg, shard = q4.shard_weights(cfg, w, 1, world)
    owned = {int(k.split(".experts.")[1].split(".")[0]) for k in shard if ".mlp.experts." in k}
    assert owned == {e for e in range(cfg.num_experts) if e % world == 1}
    assert shard["lm_head"].shape[0] == cfg.vocab_size // world and rcfg.num_heads == cfg.num_heads // world
    assert shard["layers.1.self_attn.o_proj"].shape[1] == cfg.num_heads * cfg.head_dim // world
    assert torch.equal(shard["layers.1.self_attn.index_qk_proj"], w["layers.1.self_attn.index_qk_proj"])
    assert torch.equal(shard["layers.0.attn_hc.down"], w["layers.0.attn_hc.down"])
    sizes = [sum(t.numel() for t in q4.shard_weights(cfg, w, r, world)[1].values()) for r in range(world)]
    assert max(sizes) < sum(t.numel() for t in w.values())
    with pytest.raises(AssertionError):
        q4.shard_weights(q4.Qwen4ExpConfig(), q4.synth_weights(q4.Qwen4ExpConfig(), 0), 0, 3)
