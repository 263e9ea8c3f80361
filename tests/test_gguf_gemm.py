"""GGUF blocks decoded inside the tcgen05 GEMM against the fp32 reference dequantisation."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tname", ["Q8_0", "Q4_K", "Q5_K", "Q6_K", "Q3_K", "Q2_K", "IQ1_M", "IQ2_XXS", "IQ2_XS", "IQ3_XXS", "IQ4_XS"])
@pytest.mark.parametrize("t,n,k", [(1, 256, 512), (20, 300, 1024), (200, 128, 256), (600, 512, 768), (3, 256, 4096)])
def test_gguf_linear_matches_dequantised_matmul(tname, t, n, k):
    from deepseek_v4_2080ti_b200.formats import gguf as G
    from deepseek_v4_2080ti_b200.ops import _lib, gguf_gemm
    if tname != "Q8_0" and k % 256:
        pytest.skip("k-quants need 256-wide super-blocks")
    ty = G.GGMLType[tname]
    torch.manual_seed(n + k)
    w = torch.randn(n, k, device="cuda") * 0.05
    raw = G.quantize(w, ty)
    wd = G.dequantize(raw, ty, k)
    x = torch.randn(t, k, device="cuda").bfloat16()
    r = torch.randn(t, n, device="cuda").bfloat16()
    lin = gguf_gemm.GGUFLinear.from_raw(raw, ty, n, k)
    y = gguf_gemm.linear(x, lin, residual=r)
    y32 = gguf_gemm.linear(x, lin, out_f32=True)
    torch.cuda.synchronize()
    _lib.check_status()
    ref = x.float() @ wd.bfloat16().float().t()          # the kernel rounds decoded weights to bf16
    assert ((y32 - ref).norm() / ref.norm()).item() < 5e-3
    assert ((y.float() - (ref + r.float())).norm() / (ref + r.float()).norm()).item() < 1e-2
