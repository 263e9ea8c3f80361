"""tcgen05 weight-decoding GEMM vs an fp32 PyTorch oracle (FP8 block-128 and bf16 weights)."""
import pytest
import torch

from deepseek_v4_2080ti_b200.formats import fp8 as fp8fmt

pytestmark = pytest.mark.gpu

SHAPES = [
    (1, 128, 128), (16, 128, 256), (7, 384, 512), (100, 384, 512), (33, 256, 1024),
    (300, 640, 1024), (512, 1024, 2048), (64, 5120, 1024), (257, 200, 448),
]


def _rel_err(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


@pytest.mark.parametrize("t,n,k", SHAPES)
def test_fp8_block128_matches_fp32(t, n, k):
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    torch.manual_seed(t * 1000 + n + k)
    w = torch.randn(n, k, device="cuda") * 0.05
    x = (torch.randn(t, k, device="cuda")).to(torch.bfloat16)
    q, s = fp8fmt.quantize_block128(w)
    wd = fp8fmt.dequantize_block128(q, s)
    pl = gemm.PackedLinear.from_fp8(q, s)
    y = gemm.linear(x, pl, splits=1)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = gemm.linear_ref(x, wd)
    assert _rel_err(y, ref) < 1e-2, _rel_err(y, ref)


@pytest.mark.parametrize("t,n,k", [(16, 256, 256), (200, 384, 1024), (512, 512, 512)])
def test_bf16_weights(t, n, k):
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    torch.manual_seed(0)
    w = (torch.randn(n, k, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(t, k, device="cuda").to(torch.bfloat16)
    y = gemm.linear(x, gemm.PackedLinear.from_bf16(w), splits=1)
    torch.cuda.synchronize()
    _lib.check_status()
    assert _rel_err(y, gemm.linear_ref(x, w)) < 5e-3


@pytest.mark.parametrize("t,n,k,splits", [(1, 512, 4096, 4), (8, 640, 2048, 3), (32, 256, 8192, 8)])
def test_split_k_and_residual(t, n, k, splits):
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    torch.manual_seed(1)
    w = torch.randn(n, k, device="cuda") * 0.03
    x = torch.randn(t, k, device="cuda").to(torch.bfloat16)
    r = torch.randn(t, n, device="cuda").to(torch.bfloat16)
    q, s = fp8fmt.quantize_block128(w)
    wd = fp8fmt.dequantize_block128(q, s)
    pl = gemm.PackedLinear.from_fp8(q, s)
    y = gemm.linear(x, pl, residual=r, splits=splits)
    y1 = gemm.linear(x, pl, residual=r, splits=1)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = gemm.linear_ref(x, wd, r)
    assert _rel_err(y, ref) < 1e-2
    assert _rel_err(y1, ref) < 1e-2


def test_fp32_output():
    from deepseek_v4_2080ti_b200.ops import _lib, gemm
    torch.manual_seed(2)
    w = (torch.randn(1000, 512, device="cuda") * 0.05).to(torch.bfloat16)
    x = torch.randn(5, 512, device="cuda").to(torch.bfloat16)
    y = gemm.linear(x, gemm.PackedLinear.from_bf16(w), out_f32=True)
    torch.cuda.synchronize()
    _lib.check_status()
    assert y.dtype == torch.float32
    assert _rel_err(y, gemm.linear_ref(x, w)) < 2e-3
