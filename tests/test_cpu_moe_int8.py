"""Host INT8 (W8A8) routed experts against a PyTorch statement of the same quantised arithmetic."""
import pytest
import torch
import torch.nn.functional as F

from deepseek_v4_2080ti_b200.models import mla_moe


def _q(x):
    amax = x.abs().amax(-1, keepdim=True)
    scale = amax / 127.0
    q = torch.where(amax > 0, torch.round(x / scale.clamp_min(1e-30)).clamp(-127, 127), torch.zeros_like(x))
    return q, scale.squeeze(-1)


def _oracle(x, idx, wts, w13q, s13, w2q, s2, limit):
    t, h = x.shape
    inter = w13q.shape[1] // 2
    xq, xs = _q(x)
    out = torch.zeros(t, h)
    for ti in range(t):
        for k in range(idx.shape[1]):
            e = int(idx[ti, k])
            if e < 0:
                continue
            acc = (w13q[e].double() @ xq[ti].double()).float() * (xs[ti] * s13[e])
            gate, up = acc[:inter], acc[inter:]
            if limit > 0:
                gate, up = gate.clamp(max=limit), up.clamp(-limit, limit)
            hid = wts[ti, k] * F.silu(gate) * up
            hq, hs = _q(hid[None])
            out[ti] += (w2q[e].double() @ hq[0].double()).float() * (hs[0] * s2[e])
    return out


@pytest.mark.parametrize("t,h,inter,e,k,limit", [(5, 64, 48, 6, 2, 0.0), (3, 100, 36, 4, 3, 1.5), (1, 32, 16, 2, 1, 0.0)])
def test_int8_moe_matches_the_quantised_statement_and_the_float_model(t, h, inter, e, k, limit):
    g = torch.Generator().manual_seed(t + h)
    x = torch.randn(t, h, generator=g)
    w13, w2 = torch.randn(e, 2 * inter, h, generator=g) * 0.1, torch.randn(e, h, inter, generator=g) * 0.1
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32)
    if t > 1:
        idx[1, -1] = -1                                        # an unused route
    wts = torch.rand(t, k, generator=g)
    w13q, s13 = mla_moe.quantize_rows_int8(w13)
    w2q, s2 = mla_moe.quantize_rows_int8(w2)
    rq, rs = _q(w13)
    assert torch.equal(w13q.float(), rq) and torch.allclose(s13, rs) and w13q.dtype == torch.int8
    got = mla_moe.cpu_moe_int8(x, idx, wts, w13q, s13, w2q, s2, limit, threads=3)
    want = _oracle(x, idx, wts, w13q.float(), s13, w2q.float(), s2, limit)
    assert torch.allclose(got, want, atol=2e-3 * want.abs().max().item() + 1e-6), (got - want).abs().max()
    assert torch.equal(got, mla_moe.cpu_moe_int8(x, idx, wts, w13q, s13, w2q, s2, limit, threads=1))     # thread-count invariant
    # and it is a faithful 8-bit approximation of the float experts
    ref = torch.zeros(t, h)
    for ti in range(t):
        for kk in range(k):
            ee = int(idx[ti, kk])
            if ee >= 0:
                a = w13[ee] @ x[ti]
                gt, up = a[:inter], a[inter:]
                if limit > 0:
                    gt, up = gt.clamp(max=limit), up.clamp(-limit, limit)
                ref[ti] += wts[ti, kk] * (w2[ee] @ (F.silu(gt) * up))
    assert (got - ref).abs().max() < 0.05 * ref.abs().max() + 1e-3


def test_int8_moe_rejects_bad_routes_and_handles_zero_rows():
    x = torch.zeros(2, 32)
    w13q, s13 = mla_moe.quantize_rows_int8(torch.randn(2, 32, 32))
    w2q, s2 = mla_moe.quantize_rows_int8(torch.randn(2, 32, 16))
    idx, wts = torch.tensor([[0], [1]], dtype=torch.int32), torch.ones(2, 1)
    assert torch.equal(mla_moe.cpu_moe_int8(x, idx, wts, w13q, s13, w2q, s2), torch.zeros(2, 32))
    with pytest.raises(RuntimeError):
        mla_moe.cpu_moe_int8(x, torch.tensor([[0], [5]], dtype=torch.int32), wts, w13q, s13, w2q, s2)
    zq, zs = mla_moe.quantize_rows_int8(torch.zeros(3, 8))
    assert not zq.any() and not zs.any()


@pytest.mark.parametrize("tname,k", [("Q8_0", 96), ("Q8_0", 512), ("Q2_K", 256), ("Q2_K", 768), ("IQ2_XXS", 512)])
def test_host_gguf_linear_matches_the_dequantised_product(tname, k):
    from deepseek_v4_2080ti_b200.formats.gguf import quant
    from deepseek_v4_2080ti_b200.formats.gguf.constants import GGMLType
    t = GGMLType[tname]
    g = torch.Generator().manual_seed(k)
    w = torch.randn(37, k, generator=g) * 0.3
    w[3] = 0.0                                                  # an all-zero row
    w[5] *= 1e-6                                                # scales that are subnormal in fp16
    raw = quant.quantize(w, t)
    x = torch.randn(4, k, generator=g)
    want = x @ quant.dequantize(raw, t, k).t()
    got = mla_moe.cpu_gguf_linear(x, raw, int(t), threads=3)
    assert got.shape == (4, 37) and torch.allclose(got, want, atol=1e-4 * want.abs().max().item() + 1e-7, rtol=1e-4)
    assert torch.equal(got, mla_moe.cpu_gguf_linear(x, raw, int(t), threads=1))
    with pytest.raises(RuntimeError):
        mla_moe.cpu_gguf_linear(x, raw, 12)
    with pytest.raises(RuntimeError):
        mla_moe.cpu_gguf_linear(x[:, :k - 8], raw, int(t))


def test_host_gguf_routed_experts_match_the_dequantised_experts():
    from deepseek_v4_2080ti_b200.formats.gguf import quant
    from deepseek_v4_2080ti_b200.formats.gguf.constants import GGMLType
    g = torch.Generator().manual_seed(3)
    e, h, inter, t, k = 5, 256, 256, 6, 2
    gate, up, down = (torch.randn(e, inter, h, generator=g) * 0.1, torch.randn(e, inter, h, generator=g) * 0.1,
                      torch.randn(e, h, inter, generator=g) * 0.1)
    q = lambda w, ty: torch.stack([quant.quantize(w[i], ty) for i in range(e)])
    gr, ur, dr = q(gate, GGMLType.IQ2_XXS), q(up, GGMLType.IQ2_XXS), q(down, GGMLType.Q2_K)
    dq = lambda raw, ty, cols: torch.stack([quant.dequantize(raw[i], ty, cols) for i in range(e)])
    gd, ud, dd = dq(gr, GGMLType.IQ2_XXS, h), dq(ur, GGMLType.IQ2_XXS, h), dq(dr, GGMLType.Q2_K, inter)
    x = torch.randn(t, h, generator=g)
    idx = torch.stack([torch.randperm(e, generator=g)[:k] for _ in range(t)]).to(torch.int32)
    idx[2, 1] = -1
    wts = torch.rand(t, k, generator=g)
    want = torch.zeros(t, h)
    for ti in range(t):
        for kk in range(k):
            ee = int(idx[ti, kk])
            if ee >= 0:
                a, b = (gd[ee] @ x[ti]).clamp(max=2.0), (ud[ee] @ x[ti]).clamp(-2.0, 2.0)
                want[ti] += dd[ee] @ (wts[ti, kk] * F.silu(a) * b)
    got = mla_moe.cpu_moe_gguf(x, idx, wts, gr, ur, dr, int(GGMLType.IQ2_XXS), int(GGMLType.Q2_K), swiglu_limit=2.0, threads=2)
    assert torch.allclose(got, want, atol=1e-4 * want.abs().max().item() + 1e-6, rtol=1e-3)


def test_cpu_dot_bench_reports_every_kernel(capsys):
    from deepseek_v4_2080ti_b200.utils import cpu_dot_bench
    assert cpu_dot_bench.main(["--rows", "64", "--cols", "256", "--repeat", "1", "--threads", "2"]) == 0
    import json
    rows = [json.loads(l) for l in capsys.readouterr().out.strip().splitlines()]
    assert [r["kernel"] for r in rows] == ["gguf_q8_0_gemv", "gguf_q2_k_gemv", "gguf_iq2_xxs_gemv", "int8_w8a8_moe_decode"]
    assert all(r["ms"] > 0 and r["weight_gbs"] > 0 for r in rows)
