// Op contracts of the sm_100a kernel library: plain C entry points that take raw
// device pointers and a stream and return 0 on success (a cudaError_t value or a
// negative b200 error code otherwise).  No torch type appears here, so the native
// engine executable and the torch bindings share one set of launchers.
// (Plays the role of the reference's op-contract headers,
// cpp_engine/include/{cuda_ops,qwen_ops,qwen_cuda_ops,sampler_ops}.hpp.)
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ---- GEMM (gemm_wdec.cu)
int b200_gemm_pick_bn(int T);
int b200_gemm_wdec(int wfmt, const void* W, const float* scales, const void* X, void* out_bf16,
                   float* out_f32, const void* residual, int T, int N, int K, int splits,
                   int* status, cudaStream_t stream);
int b200_splitk_reduce(const float* part, int splits, long long n, const void* residual,
                       void* out_bf16, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
