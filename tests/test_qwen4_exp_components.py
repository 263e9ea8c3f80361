"""Qwen4-Exp building blocks: MRoPE interleave, gated hyper-connection mixer + injection, hashed n-gram rows,
soft-max router, block-pooled sparse indexer."""
import torch

from deepseek_v4_2080ti_b200.models import qwen4_exp_components as q4


def test_mrope_text_only_equals_plain_rope_and_axes_interleave():
    pos = torch.arange(7)[None]
    cos, sin = q4.mrope_cos_sin(pos, 16, 10000.0, (2, 3, 3))
    inv = 1.0 / (10000.0 ** (torch.arange(0, 16, 2).float() / 16))
    want = torch.cat([pos[0, :, None] * inv, pos[0, :, None] * inv], -1)
    assert torch.allclose(cos[0], want.cos(), atol=1e-6) and torch.allclose(sin[0], want.sin(), atol=1e-6)
    p3 = torch.stack([pos, pos * 0 + 5, pos * 0 + 9])            # distinct height / width positions
    c3, _ = q4.mrope_cos_sin(p3, 16, 10000.0, (2, 3, 3))
    f = torch.acos(c3[0, 3, :8].clamp(-1, 1))
    # frequency slots 1, 4, 7 follow the height axis (position 5), 2 and 5 the width axis (9), 0, 3, 6 the text axis (3)
    ang = lambda p, i: torch.remainder(torch.tensor(p * float(inv[i])), 2 * torch.pi)
    for i, p in ((0, 3), (1, 5), (2, 9), (3, 3), (4, 5), (5, 9), (6, 3), (7, 5)):
        a = ang(p, i)
        assert torch.isclose(torch.cos(a), c3[0, 3, i], atol=1e-5), (i, p)
    x = torch.randn(1, 7, 2, 24)
    y = q4.apply_rotary_half(x, cos, sin)
    assert torch.allclose(y[..., 16:], x[..., 16:]) and torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)


def test_gated_residual_mixes_and_injects():
    torch.manual_seed(0)
    hc, h = 4, 8
    hyper = torch.randn(2, 5, hc * h)
    norm, down, up, inj = torch.rand(hc * h) + 0.5, torch.randn(6, hc * h) * 0.1, torch.randn(hc * h, 6) * 0.1, torch.randn(hc, hc * h) * 0.1
    mixed, inject = q4.gated_residual(hyper, norm, down, up, inj, hc, h)
    assert mixed.shape == (2, 5, h) and inject.shape == (2, 5, hc) and (inject > 0).all() and (inject < 2).all()
    assert q4.gated_residual(hyper, norm, down, up, None, hc, h).shape == (2, 5, h)
    out = torch.randn(2, 5, h)
    new = q4.inject_into_streams(out, hyper, inject)
    assert torch.allclose(new.unflatten(-1, (hc, h))[:, :, 2], hyper.unflatten(-1, (hc, h))[:, :, 2] + inject[:, :, 2:3] * out)
    # zero gates give a plain mean of the normalised streams weighted by sigmoid(0) = 1/2
    m0 = q4.gated_residual(hyper, torch.ones(hc * h), down * 0, up * 0, None, hc, h)
    g = hyper.unflatten(-1, (hc, h))
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + 1e-6)
    assert torch.allclose(m0, 0.5 * g.mean(-2), atol=1e-5)


def test_ngram_rows_respect_document_boundaries_and_table_slices():
    mult = q4.ngram_multipliers(1000, 3, 1, 42)
    assert mult.shape == (3,) and (mult % 2 == 1).all() and not torch.equal(mult, q4.ngram_multipliers(1000, 3, 2, 42))
    sizes, offsets = torch.tensor([101, 103, 107, 109]), torch.tensor([0, 101, 204, 311])
    eos = 0
    hist = torch.tensor([[5, 6, 7, 0, 8, 9, 5, 6, 7]])
    rows = q4.ngram_row_ids(hist, 7, 3, 2, sizes, offsets, mult, eos)
    assert rows.shape == (1, 7, 4)
    for hd in range(4):
        assert ((rows[..., hd] >= offsets[hd]) & (rows[..., hd] < offsets[hd] + sizes[hd])).all()
    # the trigram (5, 6, 7) hashes to the same rows both times it occurs; the one right after EOS does not see across it
    assert torch.equal(rows[0, 0], rows[0, 6])
    after = q4.ngram_row_ids(torch.tensor([[1, 2, 0, 8, 9]]), 1, 3, 2, sizes, offsets, mult, eos)
    same = q4.ngram_row_ids(torch.tensor([[3, 4, 0, 8, 9]]), 1, 3, 2, sizes, offsets, mult, eos)
    assert torch.equal(after, same)


def test_router_and_qsa_selection():
    torch.manual_seed(1)
    w, idx = q4.topk_softmax_router(torch.randn(5, 16), torch.randn(12, 16), 3)
    assert torch.allclose(w.sum(-1), torch.ones(5)) and idx.shape == (5, 3)
    b, s, hi, d, kv, ratio, budget = 1, 3, 2, 16, 40, 4, 16
    q = torch.randn(b, s, hi, d)
    keys = torch.randn(b, kv, d)
    cos, sin = q4.mrope_cos_sin(torch.arange(kv)[None], d, 10000.0, (2, 3, 3))
    past = kv - s
    sel = q4.qsa_select(q, keys, torch.ones(d), cos, sin, past, budget, ratio)
    assert sel.shape == (b, s, budget + ratio - 1) and sel.dtype == torch.int32
    for i in range(s):
        ids = [t for t in sel[0, i].tolist() if t >= 0]
        vis = past + i + 1
        assert len(ids) == len(set(ids)) and max(ids) < vis
        tail = list(range(vis // ratio * ratio, vis))
        assert all(t in ids for t in tail)                                   # ragged tail always visible
        assert len(ids) == budget + len(tail)
        blocks = sorted({t // ratio for t in ids if t < vis // ratio * ratio})
        assert len(blocks) == budget // ratio and all(all(bk * ratio + j in ids for j in range(ratio)) for bk in blocks)
    # short context: everything visible, causal mask only
    short = q4.qsa_select(q, keys[:, :10], torch.ones(d), cos[:, :10], sin[:, :10], 7, budget, ratio)
    assert short.shape == (1, 3, 10) and short[0, 0].tolist() == list(range(8)) + [-1, -1]
