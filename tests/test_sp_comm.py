"""Sequence-parallel residual stream on ONE GPU: the ranks of a tensor-parallel group are emulated as
``PeerComm.local_group`` communicators over symmetric buffers of the same device and stepped phase by phase on one
stream, so every flag a kernel waits for was raised by a kernel that has already completed.

Covers the reduce-scatter GEMM epilogue (gemm_wdec_kernel.cuh, ar_mode 3), the reduce + residual + RMSNorm +
all-gather kernel (comm/sp_comm.cu) and the all-gather GEMM (ag_wait) against a plain fp32 PyTorch statement of the
same math, plus the bounded-wait path: a flag that nothing sets makes the kernel return ERR_WAIT_PEER."""
import pytest
import torch

from deepseek_v4_2080ti_b200.formats import fp8 as fp8fmt

pytestmark = pytest.mark.gpu


def _bf(x):
    return x.to(torch.bfloat16)


def _ref_pipeline(xs, ws, h, gamma, eps, w2s):
    """fp32 statement with the kernels' roundings: bf16 partials, bf16 reduced projection, bf16 residual stream."""
    parts = [_bf(x.float() @ w.float().t()).float() for x, w in zip(xs, ws)]
    delta = _bf(sum(parts)).float()
    h_new = _bf(h.float() + delta)
    hf = h_new.float()
    xn = _bf(hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * (1.0 + gamma.float()))
    outs = [xn.float() @ w2.float().t() for w2 in w2s]
    return h_new, xn, outs


@pytest.mark.parametrize("world,rows,hidden,kr,fmt", [
    (2, 128, 256, 128, "bf16"), (4, 128, 384, 192, "bf16"), (8, 128, 256, 128, "bf16"),
    (2, 256, 256, 128, "bf16"), (2, 128, 256, 256, "fp8"), (4, 256, 512, 128, "fp8"),
    # many tiles per CTA pair with a short K: the epilogue warps of the pair kernel drift tiles apart
    (2, 4096, 1024, 128, "bf16"), (4, 1024, 1536, 64, "bf16"),
])
def test_reduce_scatter_norm_gather_gemm(world, rows, hidden, kr, fmt):
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    from deepseek_v4_2080ti_b200.parallel import tp

    torch.manual_seed(world * 131 + rows + hidden)
    t = world * rows
    comms = tp.PeerComm.local_group(world, slot_elems=t * hidden, budget_ms=200.0)
    assert comms[0].sp_rows(t, hidden) == rows
    n2 = 256
    xs, ws_ref, ws, w2_ref, w2s = [], [], [], [], []
    for r in range(world):
        xs.append(_bf(torch.randn(t, kr, device="cuda")))
        w = torch.randn(hidden, kr, device="cuda") * 0.05
        w2 = torch.randn(n2, hidden, device="cuda") * 0.05
        if fmt == "fp8":
            q, s = fp8fmt.quantize_block128(w)
            ws_ref.append(fp8fmt.dequantize_block128(q, s))
            ws.append(gemm.PackedLinear.from_fp8(q, s))
        else:
            ws_ref.append(_bf(w))
            ws.append(gemm.PackedLinear.from_bf16(w))
        w2_ref.append(_bf(w2))
        w2s.append(gemm.PackedLinear.from_bf16(w2))
    h_full = _bf(torch.randn(t, hidden, device="cuda"))
    gamma = _bf(torch.randn(hidden, device="cuda") * 0.1)
    eps = 1e-6
    shards = [h_full[r * rows:(r + 1) * rows].clone() for r in range(world)]

    for rep in range(2):        # twice: the second pass runs on the other parity of flags and slots
        h_before = torch.cat(shards)
        for r in range(world):
            comms[r].linear_rs(xs[r], ws[r])
        gathered = [comms[r].reduce_norm_gather(shards[r], gamma, eps, True) for r in range(world)]
        outs = []
        for r in range(world):
            outs.append(comms[r].linear_ag(gathered[r], w2s[r]))
        for r in range(world):
            comms[r].wait_gather(rows)
        torch.cuda.synchronize()
        _lib.check_status()
        h_ref, x_ref, out_ref = _ref_pipeline(xs, ws_ref, h_before, gamma, eps, w2_ref)
        h_now = torch.cat(shards)
        # bf16 partials of a tensor-core GEMM against an fp32 matmul: allow one bf16 ulp on a few elements
        # (FP8 weights are decoded to bf16 inside the kernel: one more rounding than the fp32 dequantised oracle)
        tol = 1e-2 if fmt == "fp8" else 2e-3
        assert (h_now.float() - h_ref.float()).abs().max() <= 4 * tol * h_ref.float().abs().max()
        assert ((h_now.float() - h_ref.float()).norm() / h_ref.float().norm()) < tol
        for r in range(world):
            assert torch.equal(gathered[r], gathered[0])          # every rank holds the same gathered rows
            assert ((gathered[r].float() - x_ref.float()).norm() / x_ref.float().norm()) < 2 * tol
            ref = gathered[0].float() @ w2_ref[r].float().t()
            assert ((outs[r].float() - ref).norm() / ref.norm()) < 5e-3
    for c in comms:
        c.close()


def test_norm_gather_without_partials_and_local_fold():
    """First layer (nothing to reduce yet) and the gather-free form that only folds the partials into the residual."""
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    from deepseek_v4_2080ti_b200.parallel import tp

    torch.manual_seed(3)
    world, rows, hidden, kr = 2, 128, 256, 128
    t = world * rows
    comms = tp.PeerComm.local_group(world, slot_elems=t * hidden, budget_ms=200.0)
    gamma = _bf(torch.randn(hidden, device="cuda") * 0.1)
    shards = [_bf(torch.randn(rows, hidden, device="cuda")) for _ in range(world)]
    before = [s.clone() for s in shards]
    g = [comms[r].reduce_norm_gather(shards[r], gamma, 1e-6, True, with_partials=False) for r in range(world)]
    for r in range(world):
        comms[r].wait_gather(rows)
    torch.cuda.synchronize()
    hf = torch.cat(before).float()
    ref = _bf(hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + 1e-6) * (1.0 + gamma.float()))
    assert torch.equal(torch.cat(shards), torch.cat(before))
    for r in range(world):
        assert (g[r].float() - ref.float()).abs().max() <= 2 ** -7 * ref.float().abs().max() + 1e-6
    xs = [_bf(torch.randn(t, kr, device="cuda")) for _ in range(world)]
    ws = [_bf(torch.randn(hidden, kr, device="cuda") * 0.05) for _ in range(world)]
    for r in range(world):
        comms[r].linear_rs(xs[r], gemm.PackedLinear.from_bf16(ws[r]))
    for r in range(world):
        assert comms[r].reduce_norm_gather(shards[r], None, 1e-6, True, gather=False) is None
    torch.cuda.synchronize()
    _lib.check_status()
    delta = _bf(sum(_bf(x.float() @ w.float().t()).float() for x, w in zip(xs, ws))).float()
    ref_h = _bf(torch.cat(before).float() + delta)
    assert ((torch.cat(shards).float() - ref_h.float()).norm() / ref_h.float().norm()) < 2e-3
    for c in comms:
        c.close()


def test_wait_on_a_flag_nothing_sets_returns_a_status():
    """Rank 0 of a 2-rank group runs alone: its peer never raises a flag.  The kernels give up after their (short)
    budget, write ERR_WAIT_PEER to the status word and return; the context stays usable."""
    from deepseek_v4_2080ti_b200.ops import _lib
    from deepseek_v4_2080ti_b200.parallel import tp

    comms = tp.PeerComm.local_group(2, slot_elems=1 << 16, budget_ms=5.0)
    v = torch.ones(4096, dtype=torch.bfloat16, device="cuda")
    comms[0].all_reduce(v)                         # one-shot all-reduce: waits for rank 1's push
    with pytest.raises(tp.CollectiveTimeoutError):
        comms[0].check()
    _lib.check_status()                            # the word was cleared by the failed check
    idx = torch.zeros(4, dtype=torch.int32, device="cuda")
    val = torch.ones(4, dtype=torch.float32, device="cuda")
    comms[0].argmax_merge(idx, val)
    with pytest.raises(tp.CollectiveTimeoutError):
        comms[0].check()
    # sequence-parallel gather: rank 0 waits for rank 1's partial tiles, which never come
    h = torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    g = torch.zeros(256, dtype=torch.bfloat16, device="cuda")
    comms[0]._rs_bn = 128
    comms[0].reduce_norm_gather(h, g, 1e-6, True, with_partials=True)
    comms[0].wait_gather(128)
    with pytest.raises(tp.CollectiveTimeoutError):
        comms[0].check()
    # the device is still healthy
    assert float((torch.ones(8, device="cuda") * 2).sum().item()) == 16.0
    for c in comms:
        c.close()


def test_all_gather_gemm_with_swiglu_epilogue():
    """The gathered rows feed the feed-forward block's first GEMM, which applies silu(gate) * up in its epilogue."""
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    from deepseek_v4_2080ti_b200.parallel import tp

    torch.manual_seed(11)
    world, rows, hidden, inter = 2, 1024, 256, 256
    t = world * rows
    comms = tp.PeerComm.local_group(world, slot_elems=t * hidden, budget_ms=200.0)
    gamma = _bf(torch.randn(hidden, device="cuda") * 0.1)
    shards = [_bf(torch.randn(rows, hidden, device="cuda")) for _ in range(world)]
    ws, refs = [], []
    for r in range(world):
        q, s = fp8fmt.quantize_block128(torch.randn(2 * inter, hidden, device="cuda") * 0.08)
        ws.append(gemm.PackedLinear.from_fp8(q, s))
        refs.append(_bf(fp8fmt.dequantize_block128(q, s)))
    g = [comms[r].reduce_norm_gather(shards[r], gamma, 1e-6, True, with_partials=False) for r in range(world)]
    outs = [comms[r].linear_ag_swiglu(g[r], ws[r]) for r in range(world)]
    for r in range(world):
        comms[r].wait_gather(rows)
    torch.cuda.synchronize()
    _lib.check_status()
    for r in range(world):
        gu = g[0].float() @ refs[r].float().t()
        ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
        assert outs[r].shape == (t, inter)
        assert ((outs[r].float() - ref).norm() / ref.norm()) < 5e-3
    for c in comms:
        c.close()
