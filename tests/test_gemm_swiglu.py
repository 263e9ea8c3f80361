"""Feed-forward first GEMM with the SwiGLU applied in its epilogue (ops.gemm.linear_swiglu: gate/up tiles interleaved
while the FP8 matrix is expanded, pair kernel mode 4) against the plain fp32 statement of the same math."""
import pytest
import torch

from deepseek_v4_2080ti_b200.formats import fp8 as fp8fmt

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("t,inter,k", [(2048, 256, 128), (2048, 1280, 512), (4096, 512, 320)])
def test_linear_swiglu_matches_fp32(t, inter, k):
    from deepseek_v4_2080ti_b200.ops import _lib, basic, gemm
    torch.manual_seed(t + inter + k)
    w = torch.randn(2 * inter, k, device="cuda") * 0.08
    q, s = fp8fmt.quantize_block128(w)
    wd = fp8fmt.dequantize_block128(q, s).to(torch.bfloat16)
    pl = gemm.PackedLinear.from_fp8(q, s)
    x = (torch.randn(t, k, device="cuda") * 0.7).to(torch.bfloat16)
    assert gemm.swiglu_fusable(t, pl)
    for rep in range(2):                      # second pass: the other scratch buffer
        out = gemm.linear_swiglu(x, pl)
        torch.cuda.synchronize()
        _lib.check_status()
        gu = x.float() @ wd.float().t()
        ref = torch.nn.functional.silu(gu[:, :inter]) * gu[:, inter:]
        assert out.shape == (t, inter)
        err = (out.float() - ref).norm() / ref.norm()
        assert err < 4e-3, float(err)
        assert (out.float() - ref).abs().max() <= 0.02 * ref.abs().max() + 1e-3
    # the unfused pair of kernels rounds gate and up to bf16 first: same result to bf16 accuracy
    unfused = basic.silu_mul(gemm.linear(x, pl))
    assert ((out.float() - unfused.float()).norm() / unfused.float().norm()) < 8e-3
    # prefetching the interleaved expansion on the side stream gives the same bits as expanding in place
    gemm.prefetch_bf16(pl, x.device, None, gate_up=True)
    again = gemm.linear_swiglu(x, pl)
    torch.cuda.synchronize()
    assert torch.equal(again, out)
    # a plain expansion of the same matrix right after must not pick up the interleaved copy
    plain = gemm.linear(x, pl)
    torch.cuda.synchronize()
    assert ((plain.float() - gu).norm() / gu.norm()) < 4e-3


def test_not_fusable_shapes_fall_back():
    from deepseek_v4_2080ti_b200.ops import gemm
    w = torch.randn(384, 128, device="cuda") * 0.05        # 2I = 384: not a multiple of 256
    q, s = fp8fmt.quantize_block128(w)
    pl = gemm.PackedLinear.from_fp8(q, s)
    assert not gemm.swiglu_fusable(2048, pl)
    assert not gemm.swiglu_fusable(512, gemm.PackedLinear.from_fp8(*fp8fmt.quantize_block128(torch.randn(512, 128, device="cuda"))))
    assert not gemm.swiglu_fusable(2048, gemm.PackedLinear.from_bf16(torch.randn(512, 128, device="cuda")))
