"""The allocation-free split-K GEMM entry point, called through its exported C symbol.

Some embedders of the kernel library may not call the CUDA allocator when they need a GEMM (their
memory pool already owns the device, or their serving loop forbids allocator calls after warm-up),
so ``b200_gemm_wdec_splitk_noalloc`` keeps its split-K partials in a fixed array inside the library.
This test drives that symbol with ctypes only - no wrapper of this package in between - and checks it
against the regular workspace entry point on two back-to-back calls that reuse the same scratch.
The file sorts last on purpose: a run that stops at the first failure has then run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-9)).item()


def test_noalloc_matches_workspace_entry_point_twice():
    from deepseek_v4_2080ti_b200.formats import fp8 as fp8fmt
    from deepseek_v4_2080ti_b200.ops import _lib, gemm

    L = ctypes.CDLL(str(_lib.lib_path()))
    fn = L.b200_gemm_wdec_splitk_noalloc
    fn.restype = ctypes.c_int
    L.b200_gemm_wdec_noalloc_max_floats.restype = ctypes.c_longlong
    limit = L.b200_gemm_wdec_noalloc_max_floats()
    assert limit == 4 * 1024 * 1024

    torch.manual_seed(123)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(0 if t is None else t.data_ptr())

    # two different problems in a row: the second must not be disturbed by what the first left in the scratch
    for (t, n, k, splits, use_res) in [(8, 640, 4096, 4, True), (3, 1152, 2048, 5, False)]:
        w = torch.randn(n, k, device="cuda") * 0.03
        x = torch.randn(t, k, device="cuda").to(torch.bfloat16)
        r = torch.randn(t, n, device="cuda").to(torch.bfloat16) if use_res else None
        q, s = fp8fmt.quantize_block128(w)
        pl = gemm.PackedLinear.from_fp8(q, s)
        want = gemm.linear(x, pl, residual=r, splits=splits)          # existing entry point (torch workspace)
        got = torch.empty(t, n, dtype=torch.bfloat16, device="cuda")   # caller-owned output
        rc = fn(gemm.WF_FP8_B128, p(pl.weight), p(pl.scales), p(x), p(got), p(r), t, n, k, splits, p(status), stream)
        assert rc == 0, rc
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        ref = gemm.linear_ref(x, fp8fmt.dequantize_block128(q, s), r)
        assert _rel(got, want) < 1e-2, _rel(got, want)
        assert _rel(got, ref) < 1e-2, _rel(got, ref)

    # a request larger than the built-in scratch is refused before anything is launched
    big_t, big_n, big_k, big_s = 128, 34816, 1024, 4
    assert big_t * big_n * big_s > limit
    rc = fn(gemm.WF_FP8_B128, p(None), p(None), p(None), ctypes.c_void_p(1), p(None), big_t, big_n, big_k, big_s,
            p(status), stream)
    assert rc == -7
