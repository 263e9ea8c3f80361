"""Fused decode-step kernels against the separate kernels they replace and against fp32 PyTorch."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _terms_to_float(xq, inv_c, t, terms, k):
    vals = xq.view(torch.float8_e4m3fn).float().view(t, terms, k // 4, 4)[..., [0, 2, 1, 3]].reshape(t, terms, k)
    return sum(vals[:, j] / 16.0 ** j for j in range(terms)) * inv_c[:, None]


@pytest.mark.parametrize("t,cols,terms", [(1, 256, 3), (4, 5120, 3), (8, 5120, 2), (32, 1024, 2)])
def test_rmsnorm_split_matches_fp32(t, cols, terms):
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(0)
    h = torch.randn(t, cols, device="cuda").bfloat16()
    d = torch.randn(t, cols, device="cuda").bfloat16()
    g = (torch.randn(cols, device="cuda") * 0.1).bfloat16()
    h2 = h.clone()
    out, (xq, inv_c) = basic.rmsnorm_split(h2, d, g, terms, 1e-6, True)
    resid = (h.float() + d.float()).bfloat16()
    assert torch.equal(h2, resid)
    ref = basic.rmsnorm_ref(resid, g, 1e-6, True)
    assert (out.float() - ref).abs().max() <= 0.02 * ref.abs().max()
    rec = _terms_to_float(xq, inv_c, t, terms, cols)
    tol = 3e-4 if terms == 3 else 4e-3
    assert ((rec - out.float()).abs().max(1).values / out.float().abs().max(1).values).max() < tol


@pytest.mark.parametrize("t,inter,terms", [(1, 384, 3), (5, 17408, 3), (16, 2176, 2)])
def test_silu_mul_split_matches_fp32(t, inter, terms):
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(1)
    gu = torch.randn(t, 2 * inter, device="cuda").bfloat16()
    xq, inv_c = basic.silu_mul_split(gu, terms)
    ref = torch.nn.functional.silu(gu[:, :inter].float()) * gu[:, inter:].float()
    rec = _terms_to_float(xq, inv_c, t, terms, inter)
    tol = 5e-3 if terms == 3 else 8e-3       # includes the bf16 rounding of the activation
    assert ((rec - ref).abs().max(1).values / ref.abs().max(1).values).max() < tol


@pytest.mark.parametrize("b,hv,hk,hidden", [(1, 4, 2, 256), (3, 8, 2, 512), (2, 4, 4, 256)])
def test_gdn_decode_fused_matches_separate_kernels(b, hv, hk, hidden):
    from deepseek_v4_2080ti_b200.ops import basic, gdn, gemm
    torch.manual_seed(2)
    kd, vd = hk * 128, hv * 128
    c = 2 * kd + vd
    slots = 5
    proj = (torch.randn(b, c + vd, device="cuda") * 0.5).bfloat16()
    x = torch.randn(b, hidden, device="cuda").bfloat16()
    w_ab = (torch.randn(2 * hv, hidden, device="cuda") * 0.05).bfloat16()
    a_log = torch.log(torch.rand(hv, device="cuda") * 3 + 0.5)
    dt_bias = torch.rand(hv, device="cuda") * 2 - 1
    conv_w = (torch.randn(c, 4, device="cuda") * 0.3).bfloat16()
    tails = (torch.randn(slots, 3, c, device="cuda") * 0.5).bfloat16()
    states = torch.randn(slots, hv, 128, 128, device="cuda") * 0.1
    slot_ids = torch.tensor([3, 0, 4][:b], dtype=torch.int32, device="cuda")
    gamma = (1 + torch.randn(128, device="cuda") * 0.05).bfloat16()
    # separate kernels
    t1, s1 = tails.clone(), states.clone()
    ab = gemm.linear(x, gemm.PackedLinear.from_bf16(w_ab))
    g, beta = basic.gdn_gates(ab, 0, hv, a_log, dt_bias, hv)
    mixed = basic.conv_silu_step(proj[:, :c], conv_w, t1, slot_ids)
    core = gdn.step(s1, slot_ids, mixed, 0, kd, 2 * kd, g, beta, hv, hk)
    want = basic.gated_rmsnorm(core, proj[:, c:].unflatten(1, (hv, 128)), gamma, 1e-6).view(b, vd)
    # fused
    t2, s2 = tails.clone(), states.clone()
    got = gdn.decode_fused(proj, x, w_ab, a_log, dt_bias, conv_w, t2, s2, slot_ids, gamma, hv, hk, 1e-6)
    torch.cuda.synchronize()
    assert torch.equal(t1, t2)
    assert (s1 - s2).abs().max() <= 2e-2 * s1.abs().max()
    err = (got.float() - want.float()).abs().max() / want.float().abs().max()
    assert err < 3e-2, err


def test_fused_decode_path_follows_unfused_tokens():
    from deepseek_v4_2080ti_b200.models import qwen_hybrid as qh
    cfg = qh.QwenHybridConfig.tiny(layers=4)
    state = list(qh.synth_state(cfg, 0, "cuda", std=0.05))
    outs = []
    for fused in (True, False):
        w = qh.QwenHybridWeights(cfg, iter(state), "cuda")
        rt = qh.QwenHybridRuntime(cfg, w, max_slots=2)
        assert rt.fused_decode
        rt.fused_decode = fused
        torch.manual_seed(4)
        ids = torch.randint(0, cfg.vocab_size, (120,), device="cuda", dtype=torch.int32)
        outs.append(rt.generate(ids, 12))
    agree = sum(a == b for a, b in zip(*outs))
    assert outs[0][0] == outs[1][0] and agree >= 10, outs
