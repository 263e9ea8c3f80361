"""FlashMemory: chunk retriever (oracle on CPU, kernels against the oracle on a GPU) and the host KV swap pool."""
import pytest
import torch


def _layer(heads, q_lora, hidden, cap, compressed, seed, device="cpu"):
    from deepseek_v4_2080ti_b200.components import flashmemory as fm
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sd=1.0: (torch.randn(*s, generator=g) * sd)
    keys = torch.zeros(cap, 132, dtype=torch.uint8) if compressed else torch.zeros(cap, 128)
    l = fm.ScorerLayer(r(q_lora, hidden, sd=hidden ** -0.5).bfloat16(), r(heads * 128, q_lora, sd=q_lora ** -0.5).bfloat16(),
                       1.0 + r(q_lora, sd=0.1), r(heads, hidden, sd=hidden ** -0.5).bfloat16(), keys.to(device))
    return l, g


def test_key_compression_and_reference_scoring_properties():
    from deepseek_v4_2080ti_b200.components import flashmemory as fm
    torch.manual_seed(0)
    k = torch.randn(50, 128) * torch.rand(50, 1) * 4
    packed = fm.compress_keys(k)
    assert packed.shape == (50, 132) and packed.dtype == torch.uint8
    back = fm.decompress_keys(packed)
    assert ((back - k).norm(dim=-1) / k.norm(dim=-1)).max().item() < 0.05
    inv = fm.yarn_inv_freqs(64, 10000.0, 40.0, 4096)
    assert inv.shape == (32,) and inv[0].item() == pytest.approx(1.0) and (inv[1:] < inv[:-1]).all()
    l, g = _layer(8, 64, 256, 64, True, 1)
    l.append(torch.randn(40, 128, generator=g))
    h = torch.randn(256, generator=g)
    s = fm.score_layer_ref(h, l.wq_a, l.wq_b, l.q_norm, l.weights_proj, inv, l.keys[:40], 1234)
    assert s.shape == (40,) and (s > 0).all() and (s < 1).all()
    # the Hadamard rotation is orthonormal: rotating queries and keys alike leaves q . k unchanged
    q = fm.build_query_ref(h, l.wq_a, l.wq_b, l.q_norm, inv, 1234, 1e-6)
    from deepseek_v4_2080ti_b200.models.v4_components import hadamard128_ref
    assert torch.allclose(hadamard128_ref(hadamard128_ref(q)), q, atol=1e-4)
    idx, val = fm.topk_ref(torch.tensor([0.1, 0.9, 0.9, 0.3]), 6)
    assert idx.tolist() == [1, 2, 3, 0, -1, -1] and val[0].item() == pytest.approx(0.9)


def test_retriever_on_cpu_finds_the_planted_chunk():
    from deepseek_v4_2080ti_b200.components import flashmemory as fm
    inv = fm.yarn_inv_freqs(64, 10000.0, 1.0, 0)
    layers = []
    hs = []
    for i in range(2):
        l, g = _layer(8, 64, 256, 128, i == 0, 10 + i)
        h = torch.randn(256, generator=g)
        keys = torch.randn(100, 128, generator=g) * 0.05
        q = fm.build_query_ref(h, l.wq_a, l.wq_b, l.q_norm, inv, 777, 1e-6)
        fw = l.weights_proj.float() @ h
        keys[37] = q[int(fw.argmax())] * 0.5            # aligned with the most positively weighted head
        l.append(keys)
        layers.append(l)
        hs.append(h)
    r = fm.FlashMemoryRetriever(layers, inv, chunk_tokens=4, keep=5, window_offset=1000)
    ids, rows = r.select(hs, 777)
    assert ids[0].item() == 37 and rows[0].item() == 1037 and r.n_chunks == 100
    toks = r.token_rows(ids)
    assert toks[:4].tolist() == [148, 149, 150, 151] and toks.numel() == 20
    with pytest.raises(RuntimeError):
        layers[0].append(torch.zeros(100, 128))


def test_kv_swap_pool_lru_and_contents_on_cpu():
    from deepseek_v4_2080ti_b200.runtime.kv_swap import KvSwapManager
    m = KvSwapManager(host_chunks=10, device_chunks=3, chunk_tokens=4, row_bytes=16, device="cpu")
    data = [torch.full((4, 16), i, dtype=torch.uint8) for i in range(10)]
    for i, d in enumerate(data[:8]):
        m.store(i, d, keep_resident=i == 0)
    s = m.ensure([0, 5, -1, 6])
    assert s[2].item() == -1 and len({s[0].item(), s[1].item(), s[3].item()}) == 3
    for c, slot in zip((0, 5, 6), (s[0], s[1], s[3])):
        assert torch.equal(m.dev[int(slot)], data[c])
    st = m.stats()
    assert (st["hits"], st["misses"], st["evictions"]) == (1, 2, 0)
    s2 = m.ensure([7, 5])                               # evicts chunk 0 (least recently used), keeps 5
    assert torch.equal(m.dev[int(s2[0])], data[7]) and int(s2[1]) == int(s[1]) and 0 not in m.slot_of
    assert m.stats()["evictions"] == 1
    rows = m.rows(torch.tensor([2, -1], dtype=torch.int32))
    assert rows.tolist() == [8, 9, 10, 11, -1, -1, -1, -1]
    with pytest.raises(KeyError):
        m.ensure([9])
    with pytest.raises(RuntimeError):
        m.ensure([1, 2, 3, 4])


@pytest.mark.gpu
@pytest.mark.parametrize("compressed", [True, False])
def test_retriever_kernels_match_the_oracle(compressed):
    from deepseek_v4_2080ti_b200.components import flashmemory as fm
    from deepseek_v4_2080ti_b200.ops import _lib
    inv = fm.yarn_inv_freqs(64, 10000.0, 40.0, 4096)
    heads, q_lora, hidden, n = 64, 512, 1024, 3000
    cpu_layers, gpu_layers, hs = [], [], []
    for i in range(3):
        l, g = _layer(heads, q_lora, hidden, 4096, compressed, 20 + i)
        keys = torch.randn(n, 128, generator=g) * 0.3
        l.append(keys)
        lg, _ = _layer(heads, q_lora, hidden, 4096, compressed, 20 + i, device="cuda")
        lg.append(keys)
        cpu_layers.append(l)
        gpu_layers.append(lg)
        hs.append(torch.randn(hidden, generator=g))
    ref = fm.FlashMemoryRetriever(cpu_layers, inv, keep=48, window_offset=128, use_max=True)
    dev = fm.FlashMemoryRetriever(gpu_layers, inv, keep=48, window_offset=128, use_max=True)
    pos = 123456
    want = ref.scores(hs, pos)
    got = dev.scores([h.cuda() for h in hs], pos).cpu()
    torch.cuda.synchronize()
    _lib.check_status()
    assert (got - want).abs().max().item() < 5e-3, (got - want).abs().max().item()
    ids, rows = dev.select([h.cuda() for h in hs], pos)
    ids, rows = ids.cpu(), rows.cpu()
    # the device top-k is exact on the device scores: descending, ties to the lower id
    w_idx, _ = fm.topk_ref(got, 48)
    assert ids.tolist() == w_idx.tolist() and rows.tolist() == (w_idx + 128).tolist()
    # fewer chunks than keep: padded with -1
    small = fm.FlashMemoryRetriever([gpu_layers[0]], inv, keep=48)
    gpu_layers[0].n_chunks = 10
    ids2, rows2 = small.select([hs[0].cuda()], 5)
    assert (ids2[:10] >= 0).all() and (ids2[10:] == -1).all() and (rows2[10:] == -1).all()


@pytest.mark.gpu
def test_kv_swap_pool_on_gpu_roundtrips_through_pinned_memory():
    from deepseek_v4_2080ti_b200.runtime.kv_swap import KvSwapManager
    m = KvSwapManager(host_chunks=32, device_chunks=4, chunk_tokens=64, row_bytes=1152, device="cuda")
    g = torch.Generator(device="cuda").manual_seed(0)
    data = [torch.randint(0, 256, (64, 1152), dtype=torch.uint8, device="cuda", generator=g) for _ in range(12)]
    for i, d in enumerate(data):
        m.store(i, d)
    for want in ([3, 7, 1], [7, 9, 11, 0], [3, -1, 7]):
        slots = m.ensure(want)
        torch.cuda.synchronize()
        for c, s in zip(want, slots.tolist()):
            assert (s == -1) == (c == -1)
            if c >= 0:
                assert torch.equal(m.dev[s], data[c])
    st = m.stats()
    assert st["misses"] >= 7 and st["hits"] >= 1 and st["h2d_bytes"] == st["misses"] * 64 * 1152
