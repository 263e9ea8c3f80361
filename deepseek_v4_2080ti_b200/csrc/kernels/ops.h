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

// ---- grouped GEMM + routed-expert plumbing (gemm_wdec.cu grouped mode, moe.cu)
int b200_gemm_wdec_grouped(int wfmt, const void* W, const float* scales, const void* X, void* out_bf16, int rows_total,
                           int N, int K, int groups, const void* work_table, const int* num_work, int bn, int* status,
                           cudaStream_t stream);
int b200_moe_route(const float* logits, const float* bias, int T, int E, int K, int score_fn, int norm_topk,
                   float route_scale, int* idx, float* wts, cudaStream_t stream);
int b200_moe_plan(const int* idx, int T, int K, int expert_lo, int expert_hi, int* offsets, int* route_row,
                  int* row_token, void* work13, int* n13, int m_tiles13, int bn13, void* work2, int* n2, int m_tiles2,
                  int bn2, int max_work, cudaStream_t stream);
int b200_moe_gather(const void* x, const int* row_token, const int* offsets, int EL, void* xs, int max_rows, int H,
                    cudaStream_t stream);
int b200_moe_swiglu(const void* gu, const int* offsets, int EL, void* act, int max_rows, int I, float limit,
                    cudaStream_t stream);
int b200_moe_combine(const void* y, const int* route_row, const float* wts, const void* base, void* out, int T, int K,
                     int H, cudaStream_t stream);

// ---- latent attention (attn_mla.cu)
int b200_mla_kv_append(const void* kv, const void* gamma, float eps, const int* positions, const int* slots, float theta,
                       void* cache, int T, int C, int R, const void* kidx, const void* kidx_gamma, void* idx_cache, int DI,
                       cudaStream_t stream);
int b200_mla_q_prepare(const void* q, const int* positions, float theta, void* qn_t, void* q_pe, int T, int H, int N, int R,
                       cudaStream_t stream);
int b200_mla_indexer(const void* q_idx, const float* hw, const void* idx_cache, const int* block_table, int max_blocks, int bs,
                     const int* positions, const int* seq_of_token, float* scores, int ld, int T, int HI, int DI, float scale,
                     cudaStream_t stream);
int b200_topk_rows(const float* vals, int ld, const int* n_valid, int rows, int k, int* idx, cudaStream_t stream);
int b200_mla_attention(const void* q_lat, const void* q_pe, const void* cache, const int* block_table, int max_blocks, int bs,
                       const int* positions, const int* seq_of_token, const int* sel, int nsel, void* o_lat, int T, int H, int C,
                       int R, float scale, cudaStream_t stream);
int b200_transpose_heads(const void* in, void* out, int H, int T, int D, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
