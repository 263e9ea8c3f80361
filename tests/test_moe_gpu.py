"""GPU routed-expert path: router top-k, planning, grouped FP4 / FP8 / bf16 GEMMs, combine - against fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("fn,norm", [("softmax", False), ("sigmoid", True), ("sqrtsoftplus", True)])
def test_router_matches_reference(fn, norm):
    from deepseek_v4_2080ti_b200.models import mla_moe as mm
    from deepseek_v4_2080ti_b200.ops import moe
    torch.manual_seed(0)
    t, e, k, h = 37, 256, 6, 64
    x = torch.randn(t, h, device="cuda")
    gw = torch.randn(e, h, device="cuda") * 0.3
    bias = torch.randn(e, device="cuda") * 0.05
    cfg = mm.MlaMoeConfig(num_experts=e, experts_per_token=k, score_func=fn, norm_topk=norm, route_scale=1.5)
    want_w, want_i = mm.route(cfg, x, gw, bias)
    idx, wts = moe.route((x @ gw.t()).float().contiguous(), bias, k, fn, norm, 1.5)
    assert torch.equal(idx.long().sort(1).values, want_i.sort(1).values)
    order = idx.long().argsort(1)
    worder = want_i.argsort(1)
    assert torch.allclose(wts.gather(1, order), want_w.gather(1, worder), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("fmt", ["fp4", "fp8", "bf16"])
@pytest.mark.parametrize("t", [1, 5, 70, 600])
def test_grouped_experts_match_fp32(fmt, t):
    from deepseek_v4_2080ti_b200.formats import fp4 as fp4fmt, fp8 as fp8fmt
    from deepseek_v4_2080ti_b200.models import mla_moe as mm
    from deepseek_v4_2080ti_b200.ops import _lib, moe
    torch.manual_seed(t)
    e_total, lo, el, k, h, inter = 16, 4, 8, 4, 256, 128
    x = torch.randn(t, h, device="cuda").bfloat16()
    idx = torch.stack([torch.randperm(e_total, device="cuda")[:k] for _ in range(t)]).to(torch.int32)
    wts = torch.rand(t, k, device="cuda")
    base = torch.randn(t, h, device="cuda").bfloat16()
    w1 = [torch.randn(inter, h, device="cuda") * 0.06 for _ in range(el)]
    w3 = [torch.randn(inter, h, device="cuda") * 0.06 for _ in range(el)]
    w2 = [torch.randn(h, inter, device="cuda") * 0.06 for _ in range(el)]
    if fmt == "fp4":
        q13 = [fp4fmt.quantize(torch.cat([a, b])) for a, b in zip(w1, w3)]
        q2 = [fp4fmt.quantize(a) for a in w2]
        d13 = [fp4fmt.dequantize(*q) for q in q13]
        d2 = [fp4fmt.dequantize(*q) for q in q2]
        W13 = moe.ExpertWeights.from_fp4([q[0] for q in q13], [q[1] for q in q13])
        W2 = moe.ExpertWeights.from_fp4([q[0] for q in q2], [q[1] for q in q2])
    elif fmt == "fp8":
        q13 = [fp8fmt.quantize_block128(torch.cat([a, b])) for a, b in zip(w1, w3)]
        q2 = [fp8fmt.quantize_block128(a) for a in w2]
        d13 = [fp8fmt.dequantize_block128(*q) for q in q13]
        d2 = [fp8fmt.dequantize_block128(*q) for q in q2]
        W13 = moe.ExpertWeights.from_fp8([q[0] for q in q13], [q[1] for q in q13])
        W2 = moe.ExpertWeights.from_fp8([q[0] for q in q2], [q[1] for q in q2])
    else:
        d13 = [torch.cat([a, b]).bfloat16().float() for a, b in zip(w1, w3)]
        d2 = [a.bfloat16().float() for a in w2]
        W13 = moe.ExpertWeights.from_bf16(d13)
        W2 = moe.ExpertWeights.from_bf16(d2)
    got = moe.experts_forward(x, idx, wts, W13, W2, lo, swiglu_limit=3.0, base=base)
    got2 = moe.experts_forward(x, idx, wts, W13, W2, lo, swiglu_limit=3.0, base=base)
    torch.cuda.synchronize()
    _lib.check_status()
    want = base.float().clone()
    for ti in range(t):
        for ki in range(k):
            e = int(idx[ti, ki]) - lo
            if 0 <= e < el:
                want[ti] += wts[ti, ki] * mm.swiglu(x[ti:ti + 1].float(), d13[e][:inter], d13[e][inter:], d2[e], 3.0)[0]
    err = (got.float() - want).norm() / want.norm()
    assert err < 2e-2, err
    assert torch.equal(got, got2)
