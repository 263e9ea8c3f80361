"""Guard bands (utils/canary.py): off = plain torch.empty; on = overruns on either side are reported once, with the
buffer's name, side and offset."""
import torch

from deepseek_v4_2080ti_b200.utils import canary


def test_disabled_is_plain_allocation():
    with canary.enabled(False):
        n0 = canary.live_buffers()
        t = canary.empty(4, 8, dtype=torch.bfloat16)
        assert t.shape == (4, 8) and t.dtype == torch.bfloat16 and canary.live_buffers() == n0
        assert canary.zeros((3, 2)).sum() == 0


def test_overruns_are_found_named_and_reported_once():
    with canary.enabled(True):
        a = canary.empty(10, 7, dtype=torch.float32, name="scratch A")
        b = canary.zeros(5, dtype=torch.int32, name="counters B", band=256)
        assert a.shape == (10, 7) and a.is_contiguous() and b.sum() == 0
        assert a.data_ptr() % 256 == a.untyped_storage().data_ptr() % 256      # the band keeps the alignment
        a.fill_(1.0)
        b.fill_(7)
        assert canary.verify_all() == []                                        # writing the payload is fine
        # one float past the end of A, two bytes before B
        raw_a = torch.empty(0, dtype=torch.uint8).set_(a.untyped_storage())
        off = canary.DEFAULT_BAND + a.numel() * 4
        raw_a[off:off + 4] = 0
        raw_b = torch.empty(0, dtype=torch.uint8).set_(b.untyped_storage())
        raw_b[254:256] = 1
        found = canary.verify_all()
        text = sorted(str(v) for v in found)
        assert len(found) == 2
        assert text[0].startswith("counters B: 2 byte(s) before the buffer overwritten, first at +254")
        assert text[1].startswith("scratch A: 4 byte(s) after the buffer overwritten, first at +0")
        assert canary.verify_all() == []                                        # repainted: reported once
        try:
            raw_a[0] = 3
            canary.assert_clean()
            raise SystemError("assert_clean did not raise")
        except AssertionError as e:
            assert "scratch A" in str(e) and "before" in str(e)
        n = canary.live_buffers()
        del a, raw_a
        assert canary.live_buffers() == n - 1                                   # the registry does not keep buffers alive


import pytest


@pytest.mark.gpu
def test_symmetric_buffers_carry_guard_bands():
    from deepseek_v4_2080ti_b200.parallel import tp
    with canary.enabled(True):
        comms = tp.PeerComm.local_group(2, slot_elems=1 << 14, budget_ms=50.0)
        assert comms[0]._band == tp.PeerComm.GUARD_BYTES
        # (the sequence-parallel tests run their collectives over guarded buffers: close() verifies the bands there)
        assert comms[0].verify_guards() == [] and comms[1].verify_guards() == []
        # a byte just before rank 1's buffer
        tp.PeerComm._bytes_view(comms[1]._base.value + comms[1]._band - 1, 1).fill_(0)
        bad = comms[1].verify_guards()
        assert len(bad) == 1 and "rank 1" in bad[0] and "before" in bad[0] and f"+{comms[1]._band - 1}" in bad[0]
        assert comms[1].verify_guards() == []
        for c in comms:
            c.close()


@pytest.mark.gpu
def test_kernels_leave_the_bands_of_guarded_workspaces_alone():
    from deepseek_v4_2080ti_b200.ops import gemm
    with canary.enabled(True):
        gemm._workspaces.clear()
        x = torch.randn(8, 1024, device="cuda").to(torch.bfloat16)
        w = gemm.PackedLinear.from_bf16(torch.randn(256, 1024, device="cuda") * 0.05)
        y = gemm.linear(x, w, splits=4)       # split-K: partials and tile counters live in guarded workspaces
        torch.cuda.synchronize()
        ref = x.float() @ w.weight.float().t()
        assert ((y.float() - ref).norm() / ref.norm()) < 5e-3
        assert canary.live_buffers() >= 2
        canary.assert_clean()
        gemm._workspaces.clear()
