"""DeepSeek-V4 building blocks: rotary tables (YaRN, inverse), Hadamard rotation, index tables, KV compressor
(prefill against incremental decode), routing gate with hash routing, hyper-connection mixers; GPU kernels against
the fp32 statements."""
import pytest
import torch

from deepseek_v4_2080ti_b200.models import v4_components as v4


def test_rotary_yarn_and_inverse():
    f0 = v4.yarn_inv_freq(64, 10000.0)
    f1 = v4.yarn_inv_freq(64, 10000.0, factor=16.0, original_seq_len=4096)
    assert torch.allclose(f0[0], f1[0]) and torch.allclose(f1[-1], f0[-1] / 16) and (f1 <= f0 + 1e-9).all()
    tab = v4.rotary_table(64, 50, 10000.0, 16.0, 4096)
    x = torch.randn(2, 50, 3, 64)
    y = v4.apply_rotary(x, tab)
    assert torch.allclose(v4.apply_rotary(y, tab, inverse=True), x, atol=1e-5)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4) and torch.allclose(y[:, 0], x[:, 0], atol=1e-6)


def test_hadamard_is_orthonormal_involution():
    x = torch.randn(5, 3, 128)
    y = v4.hadamard128_ref(x)
    assert torch.allclose(v4.hadamard128_ref(y), x, atol=1e-5) and torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    e = torch.zeros(128); e[0] = 1
    assert torch.allclose(v4.hadamard128_ref(e), torch.full((128,), 128 ** -0.5))


def test_index_tables():
    w = v4.window_indices(4, 6, 0)
    assert w[0].tolist() == [0, -1, -1, -1] and w[5].tolist() == [2, 3, 4, 5]
    d = v4.window_indices(4, 1, 9)
    assert sorted(d[0].tolist()) == [0, 1, 2, 3] and d[0, -1] == 9 % 4
    v = v4.window_indices(4, 2, 9)                      # 2-token verify: the first query must not see the slot of the second
    assert (10 % 4) not in v[0].tolist() and (v[0] == -1).sum() == 1
    c = v4.compressed_indices(4, 9, 0, 100)
    assert c[2].tolist() == [-1, -1] and c[3].tolist() == [100, -1] and c[8].tolist() == [100, 101]
    assert v4.compressed_indices(4, 1, 11, 7)[0].tolist() == [7, 8, 9]


@pytest.mark.parametrize("ratio", [4, 8])
def test_compressor_prefill_equals_incremental(ratio):
    torch.manual_seed(ratio)
    dim, d, rd, s = 32, 16, 8, 3 * ratio + 2
    coff = 2 if ratio == 4 else 1
    mk = lambda: v4.Compressor(wkv, wgate, ape, norm, ratio, d, rd, tab)
    wkv, wgate = torch.randn(coff * d, dim) * 0.2, torch.randn(coff * d, dim) * 0.2
    ape, norm = torch.randn(ratio, coff * d) * 0.1, torch.rand(d) + 0.5
    tab = v4.rotary_table(rd, 64, 10000.0)
    x = torch.randn(1, s, dim)
    full = mk().forward(x, 0)
    assert full.shape == (1, s // ratio, d)
    # prefill of a prefix, then token by token
    inc = mk()
    p = ratio + 1
    got = [inc.forward(x[:, :p], 0)]
    for t in range(p, s):
        o = inc.forward(x[:, t:t + 1], t)
        if o is not None:
            got.append(o)
    got = torch.cat(got, 1)
    assert torch.allclose(got, full, atol=1e-4), (got - full).abs().max()


def test_gate_bias_selects_but_does_not_weight_and_hash_routing():
    torch.manual_seed(0)
    x, w = torch.randn(6, 16), torch.randn(8, 16)
    bias = torch.zeros(8); bias[5] = 100.0
    wt, idx = v4.gate_route(x, w, bias, 2, "sqrtsoftplus", 1.5)
    assert (idx == 5).any(1).all() and torch.allclose(wt.sum(-1), torch.full((6,), 1.5), atol=1e-5)
    wt0, idx0 = v4.gate_route(x, w, None, 2, "softmax", 1.0)
    assert torch.equal(idx0, (x @ w.t()).softmax(-1).topk(2)[1]) and (wt0.sum(-1) < 1).all()
    table = torch.randint(0, 8, (50, 2), dtype=torch.int32)
    ids = torch.randint(0, 50, (6,))
    _, idh = v4.gate_route(x, w, None, 2, "sigmoid", 1.0, tid2eid=table, input_ids=ids)
    assert torch.equal(idh, table[ids].long())


def test_sinkhorn_combination_is_doubly_stochastic_and_hc_round_trip():
    torch.manual_seed(1)
    mixes = torch.randn(2, 3, 24)
    pre, post, comb = v4.hc_split_sinkhorn(mixes, torch.tensor([1.0, 0.5, 2.0]), torch.randn(24) * 0.1)
    assert torch.allclose(comb.sum(-1), torch.ones(2, 3, 4), atol=1e-3) and torch.allclose(comb.sum(-2), torch.ones(2, 3, 4), atol=1e-3)
    assert (pre > 0).all() and (post > 0).all() and (post < 2).all()
    x = torch.randn(2, 3, 4, 16)
    y, post, comb = v4.hc_pre(x, torch.randn(24, 64) * 0.1, torch.ones(3), torch.zeros(24))
    out = v4.hc_post(y, x, post, comb)
    assert y.shape == (2, 3, 16) and out.shape == x.shape
    want = post[..., None] * y[:, :, None] + torch.einsum("bsji,bsjd->bsid", comb, x)
    assert torch.allclose(out, want, atol=1e-5)


@pytest.mark.gpu
def test_gpu_kernels_match_fp32_statements():
    from deepseek_v4_2080ti_b200.ops import v4 as v4ops
    torch.manual_seed(2)
    x = torch.randn(37, 5, 128, device="cuda").bfloat16()
    assert (v4ops.hadamard128(x).float() - v4.hadamard128_ref(x.float())).abs().max() < 2e-2
    b, s, d = 2, 9, 256
    xs = torch.randn(b, s, 4, d, device="cuda").bfloat16()
    fn, scale, base = torch.randn(24, 4 * d, device="cuda") * 0.05, torch.tensor([1.0, 0.7, 1.5], device="cuda"), torch.randn(24, device="cuda") * 0.1
    y, post, comb = v4.hc_pre(xs, fn, scale, base)                       # CUDA path
    flat = xs.flatten(2).float()
    mixes = (flat @ fn.t()) * torch.rsqrt(flat.pow(2).mean(-1, keepdim=True) + 1e-6)
    pre_r, post_r, comb_r = v4.hc_split_sinkhorn(mixes, scale, base)
    y_r = (pre_r.unsqueeze(-1) * xs.float()).sum(2)
    assert torch.allclose(post, post_r, atol=1e-4) and torch.allclose(comb, comb_r, atol=1e-4)
    assert (y.float() - y_r).abs().max() < 3e-2
    out = v4.hc_post(y, xs, post, comb)
    want = post_r[..., None] * y.float()[:, :, None] + torch.einsum("bsji,bsjd->bsid", comb_r, xs.float())
    assert (out.float() - want).abs().max() < 5e-2
