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
// b200_gemm_w8a8s_allreduce (same arguments + the peer-memory communicator) is declared beside the communicator in
// gemm_w8a8s.cu: this header stays free of the communicator's types.

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
int b200_mla_attention_splitkv(const void* q_lat, const void* q_pe, const void* cache, const int* block_table, int max_blocks,
                               int bs, const int* positions, const int* seq_of_token, const int* sel, int nsel, void* o_lat,
                               int T, int H, int C, int R, float scale, float* workspace, int splits, cudaStream_t stream);
int b200_mla_indexer_mma(const void* q_idx, const float* hw, const void* idx_cache, const int* block_table, int max_blocks,
                         int bs, const int* positions, float* scores, int ld, int T, int HI, int DI, float scale,
                         cudaStream_t stream);
int b200_mla_indexer(const void* q_idx, const float* hw, const void* idx_cache, const int* block_table, int max_blocks, int bs,
                     const int* positions, const int* seq_of_token, float* scores, int ld, int T, int HI, int DI, float scale,
                     cudaStream_t stream);
int b200_topk_rows(const float* vals, int ld, const int* n_valid, int rows, int k, int* idx, cudaStream_t stream);
int b200_mla_attention(const void* q_lat, const void* q_pe, const void* cache, const int* block_table, int max_blocks, int bs,
                       const int* positions, const int* seq_of_token, const int* sel, int nsel, void* o_lat, int T, int H, int C,
                       int R, float scale, cudaStream_t stream);
int b200_transpose_heads(const void* in, void* out, int H, int T, int D, cudaStream_t stream);

// ---- sampling (sampling.cu; candidate selection by b200_topk_rows of attn_mla.cu)
int b200_sample_candidates(const float* vals, int ld, const int* idx, int K, int rows, float temperature, float top_p,
                           float min_p, const float* u, int* out_pos, float* out_prob, cudaStream_t stream);
int b200_apply_penalties(float* logits, int ld, int n, int rows, const int* counts, float repetition, float presence,
                         float frequency, cudaStream_t stream);

// ---- DeepSeek-V4 block structure (v4_ops.cu)
int b200_hadamard128(const void* x, void* y, long long rows, cudaStream_t stream);
int b200_hc_split_pre(const float* mixes, const void* x, const float* scale, const float* base, long long T, int D, int iters,
                      float eps, void* y, float* post, float* comb, cudaStream_t stream);
int b200_hc_post(const void* y, const void* residual, const float* post, const float* comb, long long T, int D, void* out,
                 cudaStream_t stream);

// ---- load-time weight preparation (prepack.cu)
unsigned long long b200_prepack_fp8_bytes(int N, int K);
int b200_prepack_fp8(const void* w_fp8, void* out, int N, int K, cudaStream_t stream);
int b200_unpack_fp8_bf16(const void* packed, const float* scales, void* out_bf16, int N, int K, cudaStream_t stream);
int b200_bf16_to_f32(const void* in, float* out, long long n, cudaStream_t stream);

// ---- row kernels (elementwise.cu), recurrent and attention kernels (gdn.cu, rope_kv.cu, attn_gqa_*.cu)
int b200_rmsnorm(void* x, const void* delta, const float* partials, int splits, const void* gamma, void* out,
                 long long rows, int cols, float eps, int unit_offset, int write_x, cudaStream_t stream);
int b200_gated_rmsnorm(const void* x, const void* gate, const void* gamma, void* out, long long nrows, int dim, float eps,
                       int heads, long long gate_ld, cudaStream_t stream);
int b200_embedding(const int* ids, const void* table, void* out, int rows, int hidden, int vocab_lo, int vocab_hi,
                   cudaStream_t stream);
int b200_silu_mul(const void* gate_up, void* out, long long rows, int inter, cudaStream_t stream);
int b200_add(void* y, const void* x, long long n, cudaStream_t stream);
int b200_conv_silu(const void* x, int ldx, const void* w, void* tail, void* y, int ldy, int T, int C, int kw,
                   int update_tail, cudaStream_t stream);
int b200_conv_silu_step(const void* x, int ldx, const void* w, void* tails, long long slot_stride, const int* slot_ids,
                        void* y, int ldy, int B, int C, int kw, cudaStream_t stream);
int b200_gdn_step(float* states, long long slot_stride, const int* slot_ids, const void* mixed, int ld, int q_off,
                  int k_off, int v_off, const float* g, const float* beta, void* out, int B, int Hv, int Hk,
                  cudaStream_t stream);
int b200_gdn_gates(const void* ab, int ld, int a_off, int b_off, const float* a_log, const float* dt_bias, float* g,
                   float* beta, long long rows, int heads, cudaStream_t stream);
int b200_argmax(const void* logits, int is_f32, int ld, int n, int rows, int index_offset, int* out_idx, float* out_val,
                cudaStream_t stream);
long long b200_gdn_workspace_floats(int T, int Hv);
int b200_gdn_use_simt_prepare(int on);
int b200_gdn_chunked(const void* mixed, int ld, int q_off, int k_off, int v_off, const float* g, const float* beta,
                     float* state, void* out, float* workspace, int T, int Hv, int Hk, cudaStream_t stream);
int b200_qk_norm_rope_append(const void* q_src, int ldq, int q_off, int q_head_stride, int gate_in_q, const void* k_src,
                             int ldk, int k_off, const void* v_src, int ldv, int v_off, const void* q_gamma,
                             const void* k_gamma, int unit_offset, float eps, const float* inv_freq, int rot, float mscale,
                             const int* positions, const int* slots, void* q_out, void* gate_out, void* k_cache,
                             void* v_cache, int block_size, int T, int Hq, int Hkv, cudaStream_t stream);
int b200_qk_sumsq(const void* proj, int ld, int q_off, int q_width, int k_off, int k_width, float* out, int T,
                  cudaStream_t stream);
int b200_qk_fullnorm_rope_append(const void* q_src, int ldq, int q_off, const void* k_src, int ldk, int k_off,
                                 const void* v_src, int ldv, int v_off, const void* q_gamma, const void* k_gamma,
                                 const float* row_ss, int q_full_width, int k_full_width, float eps, const float* inv_freq,
                                 int rot, const int* positions, const int* slots, void* q_out, void* k_cache,
                                 void* v_cache, int block_size, int T, int Hq, int Hkv, cudaStream_t stream);
int b200_gqa_prefill(const void* q, const void* k_cache, const void* v_cache, void* out, const void* gate,
                     const int* block_table, const int* q_start, const int* q_len, const int* kv_len, int batch,
                     int max_q_len, int total_q_rows, int max_blocks, int num_blocks, int block_size, int n_q_heads,
                     int n_kv_heads, float softmax_scale, int* status, cudaStream_t stream);
int b200_gqa_prefill_ex(const void* q, const void* k_cache, const void* v_cache, void* out, const void* gate,
                        const int* block_table, const int* q_start, const int* q_len, const int* kv_len, int batch,
                        int max_q_len, int total_q_rows, int max_blocks, int num_blocks, int block_size, int n_q_heads,
                        int n_kv_heads, float softmax_scale, int window, int sinks, int* status, cudaStream_t stream);
int b200_gqa_decode_ex(const void* q, const void* k_cache, const void* v_cache, void* out, const void* gate,
                       const int* block_table, const int* kv_len, float* workspace, int batch, int max_blocks, int block_size,
                       int n_q_heads, int n_kv_heads, int splits, float softmax_scale, int window, int sinks,
                       cudaStream_t stream);
int b200_gqa_decode(const void* q, const void* k_cache, const void* v_cache, void* out, const void* gate,
                    const int* block_table, const int* kv_len, float* workspace, int batch, int max_blocks,
                    int block_size, int n_q_heads, int n_kv_heads, int splits, float softmax_scale, cudaStream_t stream);
// FlashMemory retriever (flashmemory.cu): chunk scores of one scorer layer, layer ensemble, top-k, index offset
int b200_fm_score_layer(const float* hidden, const void* wq_a, const void* wq_b, const float* q_norm, const void* weights_proj,
                        const float* inv_freqs, const void* keys8, const float* keysf, float* q_scratch, float* qlora_scratch,
                        float* fused_w, float* scores, int n_chunks, int heads, int q_lora, int hidden_dim, int rope_dim,
                        float eps, long long position, int apply_sigmoid, cudaStream_t stream);
int b200_fm_ensemble(const float* layer_scores, int n_layers, int n_chunks, int stride, int use_max, float* out,
                     cudaStream_t stream);
int b200_fm_topk(const float* scores, int n_chunks, int keep, int* out_idx, float* out_val, cudaStream_t stream);
int b200_fm_write_global_indices(const int* logical, int keep, int offset, int* out, cudaStream_t stream);
// Quantised KV cache (fmt 1 = E4M3, 2 = INT8, 3 = E4M3 keys + 4-bit values with v_min) with per-(token, head) fp32
// scales (kv8.cu, attn_gqa_decode.cu)
int b200_gqa_decode_kv8(int fmt, const void* q, const void* k8, const void* v8, const float* k_scale, const float* v_scale,
                        const float* v_min, void* out, const void* gate, const int* block_table, const int* kv_len, float* workspace, int batch,
                        int max_blocks, int block_size, int n_q_heads, int n_kv_heads, int splits, float softmax_scale,
                        int window, int sinks, cudaStream_t stream);
int b200_kv8_quantize(const void* stage_k, const void* stage_v, const int* src_slots, const int* dst_slots, void* k8,
                      void* v8, float* k_scale, float* v_scale, float* v_min, int bs_src, int bs_dst, int T, int Hkv, int fmt,
                      cudaStream_t stream);
int b200_kv8_dequantize(const void* k8, const void* v8, const float* k_scale, const float* v_scale, const float* v_min,
                        const int* block_table_row, void* stage_k, void* stage_v, int bs, int n_tokens, int Hkv, int fmt,
                        cudaStream_t stream);

#ifdef __cplusplus
}
#endif
