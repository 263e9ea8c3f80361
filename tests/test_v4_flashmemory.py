"""Long-context decode of the V4 CPU runtime: compressed rows in the host pool give the same logits as rows kept in the
layer; the shared retriever's selection replaces every indexer layer's own and is what the scorer oracle says."""
import pytest
import torch

from deepseek_v4_2080ti_b200.components import flashmemory as fm
from deepseek_v4_2080ti_b200.models import v4_block_ref as v4
from deepseek_v4_2080ti_b200.models import v4_flashmemory as lc


def _ids(cfg, n, seed=1):
    return torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(seed))


def _run(m, ids, n):
    m.reset()
    return torch.cat([m.forward(ids[:n])] + [m.forward(ids[i:i + 1]) for i in range(n, ids.numel())])


@pytest.mark.parametrize("prompt", [1, 10, 23])
def test_rows_in_the_host_pool_give_the_same_logits(prompt):
    cfg = v4.V4Config(compress_ratios=(4, 8, 4), index_topk=3, max_seq_len=128)
    w = v4.synth_weights(cfg, 0)
    ids = _ids(cfg, 70)
    want = _run(v4.V4BlockRef(cfg, w), ids, prompt)
    m = lc.V4LongContextRuntime(cfg, w, swap_device_chunks=3, chunk_entries=2)
    got = _run(m, ids, prompt)
    assert torch.equal(got, want)
    st = m.swap_stats()
    # 70 tokens -> 17 entries -> 8 finished groups per layer, far more than the 3 resident slots
    assert st["misses"] > 0 and st["evictions"] > 0 and st["hits"] > 0 and st["resident"] <= 2 * 3
    assert st["d2h_bytes"] == 2 * 8 * 2 * cfg.head_dim * 4
    assert all(l.kv.shape[0] == cfg.window for l in m.indexed)           # the layers hold the window ring only
    with pytest.raises(RuntimeError, match="host pool"):
        m.snapshot()
    # a second sequence starts from an empty pool
    assert torch.equal(_run(m, ids[:30], 5), want[:30] if prompt == 5 else _run(v4.V4BlockRef(cfg, w), ids[:30], 5))
    with pytest.raises(ValueError, match="working set"):
        lc.V4LongContextRuntime(cfg, w, swap_device_chunks=2, chunk_entries=2)


def test_shared_selection_is_the_scorer_oracle_and_drives_every_indexer_layer():
    cfg = v4.V4Config(compress_ratios=(4, 8, 4), index_topk=3, max_seq_len=128)
    w, rw = v4.synth_weights(cfg, 0), lc.synth_retriever_weights(cfg, n_retrievers=2, seed=1)
    ids = _ids(cfg, 50)
    m = lc.V4LongContextRuntime(cfg, w, retrievers=rw, use_max=False)
    m.reset()
    m.forward(ids[:20])
    assert m.last_selection is None                                      # the prompt pass keeps the layers' own indexers
    seen = []
    for i in range(20, 50):
        m.forward(ids[i:i + 1])
        pick = m.last_selection
        n = i // 4
        keys = m.src.ikeys[:n]
        inv = fm.yarn_inv_freqs(cfg.rope_head_dim, cfg.compress_rope_theta, cfg.rope_factor, cfg.original_seq_len)
        per = torch.stack([fm.score_layer_ref(m.w["embed"][ids[i]], rw[f"retrievers.l{j}.wq_a.weight"], rw[f"retrievers.l{j}.wq_b.weight"],
                                              rw[f"retrievers.l{j}.q_norm_weight"], rw[f"retrievers.l{j}.weights_proj.weight"], inv,
                                              keys, i, cfg.norm_eps) for j in range(2)])
        want, _ = fm.topk_ref(per.mean(0), cfg.index_topk)
        assert pick.tolist() == want.long().tolist() and int(pick.max()) < n
        seen.append(tuple(pick.tolist()))
    assert len(set(seen)) > 1                                            # the choice moves with the token
    # the selection changes the logits relative to the layers' own indexers, and stays finite
    plain = _run(v4.V4BlockRef(cfg, w), ids, 20)
    got = _run(m, ids, 20)
    assert torch.isfinite(got).all() and torch.equal(got[:20], plain[:20]) and (got[20:] - plain[20:]).abs().max() > 1e-5
    # max and mean ensembles are both available and differ
    mx = lc.V4LongContextRuntime(cfg, w, retrievers=rw, use_max=True)
    assert (_run(mx, ids, 20) - got).abs().max() > 0


def test_with_every_entry_selected_retriever_and_indexers_agree_and_swap_composes():
    cfg = v4.V4Config(compress_ratios=(4, 4, 0), index_topk=64, max_seq_len=128, n_hash_layers=0)
    w, rw = v4.synth_weights(cfg, 3), lc.synth_retriever_weights(cfg, seed=2)
    ids = _ids(cfg, 60, 5)
    plain = _run(v4.V4BlockRef(cfg, w), ids, 12)
    # the shared selection lags the layers' own by the entry the current token completes (position 15 is the first such
    # decode step, and what it changes stays in the deeper layers' caches): equal up to there
    m = lc.V4LongContextRuntime(cfg, w, retrievers=rw, swap_device_chunks=32, chunk_entries=4)
    got = _run(m, ids, 12)
    assert torch.allclose(got[12:15], plain[12:15], atol=5e-5, rtol=1e-4) and (got[15] - plain[15]).abs().max() > 1e-5
    assert torch.equal(got[:12], plain[:12])
    out = m.generate(ids[:12], 6)
    assert len(out) == 6 and m.swap_stats()["hits"] > 0
