"""Prefix cache: key/LRU logic on CPU; on a GPU, a cache hit resumes KV blocks and recurrent state and yields the
same tokens as a cold prefill while computing fewer prompt tokens."""
import pytest
import torch

from deepseek_v4_2080ti_b200.runtime.prefix_cache import PrefixCache


def test_lookup_returns_longest_prefix_and_lru_evicts():
    released = []
    c = PrefixCache(interval=4, max_entries=2, max_bytes=1000, release_blocks=released.extend)
    a = list(range(20))
    assert c.lookup(a) is None
    assert c.boundaries(0, 10) == [4, 8] and c.boundaries(4, 9) == [8] and c.boundaries(0, 4) == []
    assert c.insert(a, 4, [1], "s4", 10)
    assert c.insert(a, 8, [1, 2], "s8", 10)
    assert not c.insert(a, 8, [1, 2], "again", 10)         # already cached
    assert not c.insert(a, 6, [1], "odd", 10)              # not a boundary
    e = c.lookup(a[:9])
    assert e.tokens == 8 and e.snapshot == "s8" and e.blocks == [1, 2]
    assert c.lookup(a[:8]).tokens == 4                     # a hit must leave at least one token to compute
    b = a[:4] + [99] * 16
    assert c.lookup(b).tokens == 4 and c.lookup([7] * 12) is None
    assert c.contains(a, 8) and not c.contains(b, 8)
    assert c.insert(b, 8, [1, 5], "b8", 10)                # third entry: the least recently used one goes
    assert len(c) == 2 and c.stats.evictions == 1 and released == [1, 2]
    assert c.lookup(a[:12]).tokens == 4
    assert not c.insert(a, 12, [1, 2, 3], "huge", 5000)    # larger than the whole budget
    c.clear()
    assert len(c) == 0 and c.bytes == 0 and sorted(released) == [1, 1, 1, 2, 5]
    assert c.stats.hits == 4 and c.stats.tokens_reused == 8 + 4 + 4 + 4 and c.stats.lookups == 6


def test_byte_budget_evicts():
    c = PrefixCache(interval=2, max_entries=10, max_bytes=25)
    t = list(range(10))
    for b in (2, 4, 6):
        c.insert(t, b, [], None, 10)
    assert len(c) == 2 and c.bytes == 20 and c.lookup(t).tokens == 6 and not c.contains(t, 2)


@pytest.mark.gpu
def test_cache_hit_equals_cold_prefill_and_skips_tokens():
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    from deepseek_v4_2080ti_b200.ops import _lib
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    w = qh.QwenHybridWeights(cfg, qh.synth_state(cfg, 0, "cuda", std=0.05), "cuda")
    gen = torch.Generator().manual_seed(5)
    shared = torch.randint(0, cfg.vocab_size, (300,), generator=gen, dtype=torch.int32)
    p1 = torch.cat([shared, torch.randint(0, cfg.vocab_size, (37,), generator=gen, dtype=torch.int32)])
    p2 = torch.cat([shared, torch.randint(0, cfg.vocab_size, (51,), generator=gen, dtype=torch.int32)])
    cold = qh.QwenHybridRuntime(cfg, w, max_slots=2, max_context=1024)
    want1, want2 = cold.generate(p1, 8), cold.generate(p2, 8)
    rt = qh.QwenHybridRuntime(cfg, w, max_slots=2, max_context=1024)
    cache = rt.enable_prefix_cache(interval=128, max_entries=4)
    free0 = len(rt.free_blocks)
    got1 = rt.generate(p1, 8)
    assert got1 == want1 and rt.prefill_tokens_computed == p1.numel() and len(cache) == 2     # snapshots at 128, 256
    held = free0 - len(rt.free_blocks)
    assert held == 256 // rt.block_size                    # the cache keeps the prefix blocks alive
    got2 = rt.generate(p2, 8)
    torch.cuda.synchronize()
    _lib.check_status()
    assert got2 == want2
    assert rt.prefill_tokens_computed == p1.numel() + (p2.numel() - 256) and cache.stats.hits == 1
    again = rt.generate(p1, 8)                             # same prompt: resumes at 256 again
    assert again == want1
    cache.clear()
    assert len(rt.free_blocks) == free0 and all(r == 0 for r in rt.block_refs)
