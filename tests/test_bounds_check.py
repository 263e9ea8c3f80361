"""Debug index checks (B200_BOUNDS_CHECK=1, csrc/kernels/bounds.cu): an index outside its range is recorded in the
device error word with the site and the element, and replaced by a valid one before the kernel that uses it runs -
the failure is a status, the memory access stays in range."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_bad_indices_become_a_status_and_are_made_safe(monkeypatch):
    from deepseek_v4_2080ti_b200.ops import _lib
    monkeypatch.setenv("B200_BOUNDS_CHECK", "1")
    idx = torch.tensor([0, 5, 99, -1, 7, -3], dtype=torch.int32, device="cuda")
    _lib.check_indices(idx, 0, 10, 5, keep=-1)
    torch.cuda.synchronize()
    assert idx.tolist() == [0, 5, 0, -1, 7, 0]            # 99 and -3 replaced by the lower bound, the sentinel kept
    with pytest.raises(_lib.KernelError, match=r"index out of range in selected key rows at element (2|5)"):
        _lib.check_status()
    _lib.check_status()                                    # cleared
    good = torch.arange(8, dtype=torch.int32, device="cuda")
    _lib.check_indices(good, 0, 8, 3)
    _lib.check_status()
    assert good.tolist() == list(range(8))


def test_checks_are_off_by_default(monkeypatch):
    from deepseek_v4_2080ti_b200.ops import _lib
    monkeypatch.delenv("B200_BOUNDS_CHECK", raising=False)
    idx = torch.tensor([123], dtype=torch.int32, device="cuda")
    _lib.check_indices(idx, 0, 10, 1)
    torch.cuda.synchronize()
    assert idx.tolist() == [123]
    _lib.check_status()


def test_state_slot_out_of_range_is_caught_before_the_gdn_step(monkeypatch):
    """A decode step addressing recurrent state 9 of 2: with the checks on the kernel runs on slot 0 instead and the
    host gets the error.  The two states are the head of a 16-state allocation, so even an unchecked index 9 would
    land in memory this test owns; state 9 must come out untouched."""
    from deepseek_v4_2080ti_b200.ops import _lib, gdn
    from deepseek_v4_2080ti_b200.utils import canary
    monkeypatch.setenv("B200_BOUNDS_CHECK", "1")
    hv, hk = 4, 2
    with canary.enabled(True):
        big = canary.zeros(16, hv, 128, 128, dtype=torch.float32, device="cuda", name="test states")
        states = big[:2]
        ld = 2 * hk * 128 + hv * 128
        mixed = (torch.randn(1, ld, device="cuda") * 0.1).to(torch.bfloat16)
        g = torch.full((1, hv), -0.1, device="cuda")
        beta = torch.full((1, hv), 0.5, device="cuda")
        slots = torch.tensor([9], dtype=torch.int32, device="cuda")
        out = gdn.step(states, slots, mixed, 0, hk * 128, 2 * hk * 128, g, beta, hv, hk)
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all() and slots.tolist() == [0]
        with pytest.raises(_lib.KernelError, match="state slots"):
            _lib.check_status()
        assert states[0].abs().sum() > 0 and big[1:].abs().sum() == 0
        canary.assert_clean()
