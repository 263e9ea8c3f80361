"""Hot-expert cache: LRU residency over host slabs, never evicting what the same call needs; a routed MoE computed from
cached slots equals the one computed from the full weights."""
import pytest
import torch
import torch.nn.functional as F

from deepseek_v4_2080ti_b200.components.expert_cache import HotExpertCache, pack_slabs, view_slab


def _experts(n=6, d=16, inter=24, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [[torch.randn(inter, d, generator=g).to(torch.bfloat16), torch.randn(inter, d, generator=g).to(torch.bfloat16),
             torch.randn(d, inter, generator=g).to(torch.bfloat16)] for _ in range(n)]


def test_pack_and_view_round_trip():
    ex = _experts()
    slabs, layout = pack_slabs(ex)
    assert slabs.dtype == torch.uint8 and slabs.shape[0] == 6 and all(o % 16 == 0 for o, _, _ in layout)
    for e in range(6):
        for a, b in zip(view_slab(slabs[e], layout), ex[e]):
            assert torch.equal(a, b)


def test_lru_residency_hits_misses_and_pinning_of_the_current_request():
    slabs, _ = pack_slabs(_experts())
    c = HotExpertCache(slabs, capacity=3)
    s = c.fetch([0, 1, 2])
    assert s.dtype == torch.int32 and sorted(s.tolist()) == [0, 1, 2] and c.stats.misses == 3 and c.stats.hits == 0
    for e in (0, 1, 2):
        assert torch.equal(c.slab(e), slabs[e])
    c.fetch([0])                                               # 0 becomes most recent: order is 1, 2, 0
    c.fetch([3])                                               # evicts 1
    assert set(c.resident()) == {2, 0, 3} and c.stats.evictions == 1
    c.fetch([1, 2])                                            # 2 is needed by this call, so 0 goes instead
    assert set(c.resident()) == {3, 1, 2} and torch.equal(c.slab(1), slabs[1])
    assert c.stats.hits == 2 and c.stats.misses == 5 and c.stats.bytes_copied == 5 * slabs.shape[1]
    assert 0 < c.stats.hit_rate < 1
    assert c.fetch([2, 2, 3]).tolist()[0] == c.fetch([2]).tolist()[0]
    with pytest.raises(RuntimeError):
        c.fetch([0, 1, 2, 3])
    with pytest.raises(IndexError):
        c.fetch([9])
    with pytest.raises(RuntimeError):
        c.remap(torch.tensor([5]))
    assert HotExpertCache(slabs, capacity=99).capacity == 6


def test_routed_moe_through_the_cache_matches_full_weights():
    ex = _experts(n=8)
    slabs, layout = pack_slabs(ex)
    cache = HotExpertCache(slabs, capacity=4)
    g = torch.Generator().manual_seed(5)
    for step in range(6):                                      # decode-like steps: 2 tokens x top-2 experts
        x = torch.randn(2, 16, generator=g)
        idx = torch.stack([torch.randperm(8, generator=g)[:2] for _ in range(2)])
        wts = torch.rand(2, 2, generator=g)
        want = torch.zeros(2, 16)
        for t in range(2):
            for k in range(2):
                w1, w3, w2 = [m.float() for m in ex[int(idx[t, k])]]
                want[t] += wts[t, k] * ((F.silu(x[t] @ w1.t()) * (x[t] @ w3.t())) @ w2.t())
        needed = sorted(set(idx.flatten().tolist()))
        cache.fetch(needed)
        slot_idx = cache.remap(idx)
        got = torch.zeros(2, 16)
        for t in range(2):
            for k in range(2):
                w1, w3, w2 = [m.float() for m in view_slab(cache.slots[int(slot_idx[t, k])], layout)]
                got[t] += wts[t, k] * ((F.silu(x[t] @ w1.t()) * (x[t] @ w3.t())) @ w2.t())
        assert torch.allclose(got, want, atol=1e-5)
    assert cache.stats.hits + cache.stats.misses >= 12 and cache.stats.evictions > 0
