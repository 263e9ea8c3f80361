"""bf16 GEMM on CTA pairs (tcgen05.mma.cta_group::2, csrc/kernels/gemm_bf16_2cta.cu) against an fp32 PyTorch matmul,
and against the one-CTA kernel it replaces for prefill-sized problems."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("t,n,k", [(256, 256, 64), (256, 512, 256), (512, 256, 1024), (2048, 768, 512),
                                   (4096, 5120, 2048), (8192, 1536, 5120)])
def test_pair_gemm_matches_fp32(t, n, k):
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    L = _lib.lib()
    was = L.b200_gemm_2cta_enabled()
    L.b200_gemm_2cta_enable(1)
    assert L.b200_gemm_2cta_supported(t, n, k) == 1
    torch.manual_seed(t + n + k)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(t, k, device="cuda").to(torch.bfloat16)
    pl = gemm.PackedLinear.from_bf16(w)
    L.b200_gemm_2cta_enable(1)
    y2 = gemm.linear(x, pl, splits=1)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = x.float() @ w.float().t()
    assert _rel(y2, ref) < 5e-3, _rel(y2, ref)
    L.b200_gemm_2cta_enable(0)
    try:
        y1 = gemm.linear(x, pl, splits=1)
        torch.cuda.synchronize()
    finally:
        L.b200_gemm_2cta_enable(1)
    # same products, same K order, fp32 accumulation in both: the two kernels agree to the last bf16 bit almost
    # everywhere
    assert (y1.float() - y2.float()).abs().max() <= 2 ** -7 * ref.abs().max()
    # a second launch on the same buffers (barrier phases, accumulator buffers start over)
    y3 = gemm.linear(x, pl, splits=1)
    torch.cuda.synchronize()
    L.b200_gemm_2cta_enable(was)
    assert torch.equal(y2, y3)


def test_shapes_that_do_not_tile_fall_back():
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    L = _lib.lib()
    assert L.b200_gemm_2cta_supported(300, 256, 64) == 0 and L.b200_gemm_2cta_supported(256, 384, 64) == 0
    w = (torch.randn(384, 128, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(300, 128, device="cuda").to(torch.bfloat16)
    y = gemm.linear(x, gemm.PackedLinear.from_bf16(w), splits=1)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel(y, x.float() @ w.float().t()) < 5e-3
