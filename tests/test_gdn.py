"""Gated DeltaNet: chunked scan and decode step vs the fp32 token-by-token recurrence."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(t, hk, hv, seed=0):
    torch.manual_seed(seed)
    ld = 2 * hk * 128 + hv * 128
    mixed = torch.randn(t, ld, device="cuda").bfloat16()
    g = -torch.rand(t, hv, device="cuda") * 0.5
    beta = torch.rand(t, hv, device="cuda")
    state = torch.randn(hv, 128, 128, device="cuda") * 0.1
    return mixed, g, beta, state


def _split(mixed, hk, hv):
    t = mixed.shape[0]
    q = mixed[:, :hk * 128].view(t, hk, 128)
    k = mixed[:, hk * 128:2 * hk * 128].view(t, hk, 128)
    v = mixed[:, 2 * hk * 128:].view(t, hv, 128)
    return q, k, v


@pytest.mark.parametrize("t,hk,hv", [(64, 1, 1), (1, 2, 4), (100, 2, 4), (257, 2, 2), (640, 1, 2)])
def test_chunked_matches_recurrence(t, hk, hv):
    from deepseek_v4_2080ti_b200.ops import gdn
    mixed, g, beta, state = _inputs(t, hk, hv, t)
    q, k, v = _split(mixed, hk, hv)
    want_o, want_s = gdn.recurrent_ref(q, k, v, g, beta, state)
    s = state.clone()
    out = gdn.chunked(mixed, 0, hk * 128, 2 * hk * 128, g, beta, s, hv, hk)
    assert (out.float() - want_o).abs().max().item() < 2e-2 * max(1.0, want_o.abs().max().item())
    assert (s - want_s).abs().max().item() < 2e-3 * max(1.0, want_s.abs().max().item())


def test_tensor_core_prepare_tracks_the_scalar_prepare():
    """The m16n8k16 chunk preparation (fp16 operands) against the fp32 scalar kernel on the same inputs, ragged tail
    and several heads included."""
    from deepseek_v4_2080ti_b200.ops import gdn
    mixed, g, beta, state = _inputs(1000, 2, 4, 11)
    s_mma, s_simt = state.clone(), state.clone()
    o_mma = gdn.chunked(mixed, 0, 256, 512, g, beta, s_mma, 4, 2)
    was = gdn.use_simt_prepare(True)
    try:
        o_simt = gdn.chunked(mixed, 0, 256, 512, g, beta, s_simt, 4, 2)
    finally:
        gdn.use_simt_prepare(was)
    torch.cuda.synchronize()
    scale = max(1.0, o_simt.float().abs().max().item())
    assert (o_mma.float() - o_simt.float()).abs().max().item() < 1e-2 * scale
    assert (s_mma - s_simt).abs().max().item() < 2e-3 * max(1.0, s_simt.abs().max().item())


def test_two_calls_equal_one():
    from deepseek_v4_2080ti_b200.ops import gdn
    mixed, g, beta, state = _inputs(200, 2, 4, 3)
    s1 = state.clone()
    o1 = gdn.chunked(mixed, 0, 256, 512, g, beta, s1, 4, 2)
    s2 = state.clone()
    oa = gdn.chunked(mixed[:72], 0, 256, 512, g[:72].contiguous(), beta[:72].contiguous(), s2, 4, 2)
    ob = gdn.chunked(mixed[72:], 0, 256, 512, g[72:].contiguous(), beta[72:].contiguous(), s2, 4, 2)
    assert (torch.cat([oa, ob]).float() - o1.float()).abs().max().item() < 2e-2
    assert (s1 - s2).abs().max().item() < 2e-3


def test_step_matches_recurrence():
    from deepseek_v4_2080ti_b200.ops import gdn
    hk, hv, b = 2, 4, 3
    mixed, g, beta, _ = _inputs(b, hk, hv, 7)
    states = torch.randn(5, hv, 128, 128, device="cuda") * 0.1
    slots = torch.tensor([4, 0, 2], dtype=torch.int32, device="cuda")
    q, k, v = _split(mixed, hk, hv)
    want = []
    want_states = states.clone()
    for i in range(b):
        o, s = gdn.recurrent_ref(q[i:i + 1], k[i:i + 1], v[i:i + 1], g[i:i + 1], beta[i:i + 1], states[slots[i]])
        want.append(o)
        want_states[slots[i]] = s
    out = gdn.step(states, slots, mixed, 0, hk * 128, 2 * hk * 128, g, beta, hv, hk)
    assert (out.float() - torch.cat(want)).abs().max().item() < 2e-2
    assert (states - want_states).abs().max().item() < 1e-3
