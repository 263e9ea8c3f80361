"""Row kernels vs fp32 oracles."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(a, b, tol=2e-2):
    a, b = a.float(), b.float()
    assert (a - b).abs().max().item() <= tol * max(1.0, b.abs().max().item()), (a - b).abs().max().item()


@pytest.mark.parametrize("rows,cols,unit", [(1, 128, False), (7, 5120, True), (33, 3072, False), (4, 6144, True)])
def test_rmsnorm(rows, cols, unit):
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device="cuda").bfloat16()
    g = (torch.randn(cols, device="cuda") * 0.1).bfloat16()
    _close(basic.rmsnorm(x, g, 1e-6, unit), basic.rmsnorm_ref(x, g, 1e-6, unit))


def test_add_rmsnorm_with_partials():
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(1)
    rows, cols, splits = 5, 1024, 3
    r = torch.randn(rows, cols, device="cuda").bfloat16()
    d = torch.randn(rows, cols, device="cuda").bfloat16()
    parts = torch.randn(splits, rows, cols, device="cuda")
    g = (torch.randn(cols, device="cuda") * 0.1).bfloat16()
    want_r = (r.float() + d.float() + parts.sum(0)).bfloat16()
    want = basic.rmsnorm_ref(want_r, g, 1e-6, True)
    got = basic.add_rmsnorm(r, d, g, 1e-6, True, partials=parts, splits=splits)
    _close(r, want_r)
    _close(got, want)


def test_gated_rmsnorm_and_gating():
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(2)
    x = torch.randn(11, 6, 128, device="cuda").bfloat16()
    z = torch.randn(11, 6, 128, device="cuda").bfloat16()
    g = torch.randn(128, device="cuda").bfloat16()
    _close(basic.gated_rmsnorm(x, z, g), basic.gated_rmsnorm_ref(x, z, g))
    gu = torch.randn(9, 512, device="cuda").bfloat16()
    _close(basic.silu_mul(gu), basic.silu_mul_ref(gu))
    a = torch.randn(9, 256, device="cuda").bfloat16()
    b = torch.randn(9, 256, device="cuda").bfloat16()
    _close(basic.sigmoid_mul(a, b), a.float() * torch.sigmoid(b.float()))


def test_embedding_shard_and_argmax():
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(3)
    table = torch.randn(100, 256, device="cuda").bfloat16()
    ids = torch.tensor([0, 5, 99, 150, 42], dtype=torch.int32, device="cuda")
    out = basic.embedding(ids, table[40:], 40, 100)
    want = torch.zeros(5, 256, device="cuda").bfloat16()
    want[2] = table[99]
    want[4] = table[42]
    assert torch.equal(out, want)
    logits = torch.randn(6, 5000, device="cuda")
    idx, val = basic.argmax(logits, 7, True)
    assert torch.equal(idx.long(), logits.argmax(-1) + 7)
    assert torch.equal(val, logits.max(-1).values)
    assert torch.equal(basic.argmax(logits.bfloat16()).long(), logits.bfloat16().float().argmax(-1))


@pytest.mark.parametrize("t", [1, 5, 64, 200])
def test_conv_silu_chunks_and_step(t):
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(4)
    c = 512
    x = torch.randn(t, c, device="cuda").bfloat16()
    w = torch.randn(c, 4, device="cuda").bfloat16()
    tail = torch.randn(3, c, device="cuda").bfloat16()
    want, want_tail = basic.conv_silu_ref(x, w, tail)
    tail1 = tail.clone()
    _close(basic.conv_silu(x, w, tail1), want)
    assert torch.equal(tail1, want_tail)
    # token-by-token with the step kernel gives the same stream
    tails = tail.clone()[None].repeat(2, 1, 1).contiguous()
    slot = torch.tensor([1], dtype=torch.int32, device="cuda")
    ys = [basic.conv_silu_step(x[i:i + 1], w, tails, slot) for i in range(min(t, 8))]
    _close(torch.cat(ys), want[:min(t, 8)])


def test_gdn_gates():
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(5)
    ab = torch.randn(13, 64, device="cuda").bfloat16()
    a_log = torch.randn(32, device="cuda")
    dtb = torch.randn(32, device="cuda")
    g, beta = basic.gdn_gates(ab, 0, 32, a_log, dtb, 32)
    wg, wb = basic.gdn_gates_ref(ab[:, :32], ab[:, 32:], a_log, dtb)
    _close(g, wg, 1e-3)
    _close(beta, wb, 1e-3)


def test_argmax_two_stage_wide_vocabulary():
    """Few rows over a wide vocabulary go through the chunked two-launch arg-max; ties resolve to the lowest index."""
    from deepseek_v4_2080ti_b200.ops import basic
    torch.manual_seed(11)
    logits = torch.randn(3, 151936, device="cuda")
    logits[1, 70000] = logits[1, 140000] = 50.0
    idx, val = basic.argmax(logits, 1000, True)
    assert idx.tolist() == [int(logits[0].argmax()) + 1000, 71000, int(logits[2].argmax()) + 1000]
    assert torch.equal(val, logits.max(-1).values)
