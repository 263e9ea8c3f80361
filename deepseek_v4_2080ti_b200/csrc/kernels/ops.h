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
int b200_gemm_wdec_ex(int wfmt, const void* W, const float* scales, const void* X, void* out_bf16,
                      float* out_f32, const void* residual, int T, int N, int K, int splits,
                      int* tile_counters, int* status, cudaStream_t stream);
int b200_splitk_reduce(const float* part, int splits, long long n, const void* residual,
                       void* out_bf16, cudaStream_t stream);

// ---- weight-streaming FP8 GEMM for T <= 32 (gemm_w8a8s.cu)
int b200_gemm_w8a8s_layout(int T, int* terms);
int b200_act_split_e4m3(const void* x_bf16, int T, int K, int terms, void* xq, float* inv_c, cudaStream_t stream);
int b200_gemm_w8a8s(const void* W, const float* scales, const void* xq, const float* inv_c, void* out_bf16,
                    const void* residual, int T, int N, int K, int splits, float* partial, int* tile_counters,
                    int* status, cudaStream_t stream);

// ---- fused decode-step kernels (decode_fused.cu)
int b200_gdn_decode_fused(const void* proj, int ldp, const void* x, int hidden, const void* w_ab, const float* a_log,
                          const float* dt_bias, const void* conv_w, int kw, void* tails, long long tail_stride,
                          float* states, long long state_stride, const int* slot_ids, const void* gamma, void* out,
                          int B, int Hv, int Hk, float eps, cudaStream_t stream);
int b200_rmsnorm_split(void* x, const void* delta, const void* gamma, void* out, void* xq, float* inv_c, int T,
                       int cols, float eps, int unit_offset, int terms, cudaStream_t stream);
int b200_silu_mul_split(const void* gu, void* xq, float* inv_c, int T, int inter, int terms, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
