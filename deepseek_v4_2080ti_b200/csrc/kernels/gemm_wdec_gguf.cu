// Entry points of the weight-decoding GEMM for GGUF block-quantised weights (Q8_0, Q4_K, Q5_K, Q6_K, Q3_K, Q2_K, IQ1_M, IQ2_XXS, IQ2_XS, IQ3_XXS, IQ4_XS): the raw
// blocks are decoded in registers by the decode warps of gemm_wdec_kernel.cuh into bf16 tensor-core tiles; no
// dequantised copy of a weight matrix ever exists in memory.
// Reference behaviour covered: the fused dequant GEMV / GEMM family for GGUF tensors
// (src/csrc/cuda_kernel_impl.cu:6432-6700 gguf_quant_gemm*, :7039-8065 gguf_moe_*; cpp_engine/backends/cuda/kernels/
// q2_ops.cu, quant_gemm.cu), which run on dp4a / CUDA cores.
#include "gemm_wdec_kernel.cuh"

using namespace b200;

namespace {

template <int WFMT>
int dispatch_bn(int bn, const CUtensorMap& tmX, const GemmParams& p, cudaStream_t stream) {
  switch (bn) {
    case 16: return launch_one<16, WFMT>(tmX, tmX, p, stream);
    case 32: return launch_one<32, WFMT>(tmX, tmX, p, stream);
    case 64: return launch_one<64, WFMT>(tmX, tmX, p, stream);
    case 128: return launch_one<128, WFMT>(tmX, tmX, p, stream);
    case 256:
      // A decode group may run up to GROUPS k-blocks ahead of the MMA warp; its parity wait on a raw stage is only
      // sound when the ring is at least that deep (Q8_0 with 256-row activation tiles fits 3 stages only).
      if constexpr (SmemLayout<256, WFMT>::SR >= SmemLayout<256, WFMT>::GROUPS) return launch_one<256, WFMT>(tmX, tmX, p, stream);
      else return -ERR_BAD_ARG;
  }
  return -ERR_BAD_ARG;
}

bool bn256_ok(int wfmt) {
  switch (wfmt) {
    case WF_Q8_0: return SmemLayout<256, WF_Q8_0>::SR >= SmemLayout<256, WF_Q8_0>::GROUPS;
    case WF_Q4_K: return SmemLayout<256, WF_Q4_K>::SR >= SmemLayout<256, WF_Q4_K>::GROUPS;
    case WF_Q2_K: return SmemLayout<256, WF_Q2_K>::SR >= SmemLayout<256, WF_Q2_K>::GROUPS;
    case WF_IQ2_XXS: return SmemLayout<256, WF_IQ2_XXS>::SR >= SmemLayout<256, WF_IQ2_XXS>::GROUPS;
    case WF_Q5_K: return SmemLayout<256, WF_Q5_K>::SR >= SmemLayout<256, WF_Q5_K>::GROUPS;
    case WF_IQ3_XXS: return SmemLayout<256, WF_IQ3_XXS>::SR >= SmemLayout<256, WF_IQ3_XXS>::GROUPS;
    case WF_IQ1_M: return SmemLayout<256, WF_IQ1_M>::SR >= SmemLayout<256, WF_IQ1_M>::GROUPS;
    case WF_Q6_K: return SmemLayout<256, WF_Q6_K>::SR >= SmemLayout<256, WF_Q6_K>::GROUPS;
    case WF_Q3_K: return SmemLayout<256, WF_Q3_K>::SR >= SmemLayout<256, WF_Q3_K>::GROUPS;
    case WF_IQ4_XS: return SmemLayout<256, WF_IQ4_XS>::SR >= SmemLayout<256, WF_IQ4_XS>::GROUPS;
    case WF_IQ2_XS: return SmemLayout<256, WF_IQ2_XS>::SR >= SmemLayout<256, WF_IQ2_XS>::GROUPS;
  }
  return false;
}

int dispatch(int wfmt, int bn, const CUtensorMap& tmX, const GemmParams& p, cudaStream_t stream) {
  switch (wfmt) {
    case WF_Q8_0: return dispatch_bn<WF_Q8_0>(bn, tmX, p, stream);
    case WF_Q4_K: return dispatch_bn<WF_Q4_K>(bn, tmX, p, stream);
    case WF_Q2_K: return dispatch_bn<WF_Q2_K>(bn, tmX, p, stream);
    case WF_IQ2_XXS: return dispatch_bn<WF_IQ2_XXS>(bn, tmX, p, stream);
    case WF_Q5_K: return dispatch_bn<WF_Q5_K>(bn, tmX, p, stream);
    case WF_IQ3_XXS: return dispatch_bn<WF_IQ3_XXS>(bn, tmX, p, stream);
    case WF_IQ1_M: return dispatch_bn<WF_IQ1_M>(bn, tmX, p, stream);
    case WF_Q6_K: return dispatch_bn<WF_Q6_K>(bn, tmX, p, stream);
    case WF_Q3_K: return dispatch_bn<WF_Q3_K>(bn, tmX, p, stream);
    case WF_IQ4_XS: return dispatch_bn<WF_IQ4_XS>(bn, tmX, p, stream);
    case WF_IQ2_XS: return dispatch_bn<WF_IQ2_XS>(bn, tmX, p, stream);
  }
  return -ERR_BAD_ARG;
}

bool fill(GemmParams& p, int wfmt, const void* W, const void* lut, void* out_bf16, float* out_f32, const void* residual,
          int T, int N, int K, int* status) {
  if (T <= 0 || N <= 0 || K <= 0 || (K % 64) != 0 || gguf_qb(wfmt) == 0) return false;
  if ((wfmt == WF_IQ2_XXS || wfmt == WF_IQ3_XXS || wfmt == WF_IQ1_M || wfmt == WF_IQ4_XS || wfmt == WF_IQ2_XS) && !lut) return false;
  memset(&p, 0, sizeof(p));
  p.T = T; p.N = N; p.K = K;
  p.m_tiles = (N + BM - 1) / BM;
  p.n_tiles = 1;
  p.kb_total = K / BK;
  p.splits = 1;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.out_f32 = out_f32;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldo = N;
  p.status = status;
  p.w_tiled = reinterpret_cast<const uint8_t*>(W);
  p.lut = reinterpret_cast<const uint8_t*>(lut);
  return true;
}

}  // namespace

// Bytes of one (128-row, 64-input) stage of a packed GGUF weight, 0 for an unsupported format.
extern "C" int b200_gguf_stage_bytes(int wfmt) { return raw_stage_bytes(wfmt); }

// Largest activation-tile height (rows per work item of the grouped form) a format supports: 256 or 128.
extern "C" int b200_gguf_max_bn(int wfmt) { return bn256_ok(wfmt) ? 256 : 128; }

// Y[T, N] = X[T, K] W^T with W packed tile-major: [ceil(N/128)][K/64][stage bytes] (formats above; K % 64 == 0).
// Writes bf16 `out` (+ residual) or, when out_bf16 is null, fp32 `out_f32`.  lut: the codebook table of the IQ formats (IQ2_XXS: 256 x 8 magnitudes + 128 sign bytes; IQ3_XXS: 256 x 4
// magnitudes + 128 sign bytes; IQ1_M: 2048 x 8 int8).
extern "C" int b200_gemm_wdec_gguf(int wfmt, const void* W, const void* lut, const void* X, void* out_bf16, float* out_f32,
                                   const void* residual, int T, int N, int K, int* status, cudaStream_t stream) {
  GemmParams p;
  if (!fill(p, wfmt, W, lut, out_bf16, out_f32, residual, T, N, K, status) || (!out_bf16 && !out_f32)) return -ERR_BAD_ARG;
  int BN = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
  if (BN == 256 && !bn256_ok(wfmt)) BN = 128;
  p.n_tiles = (T + BN - 1) / BN;
  CUtensorMap tmX;
  if (!make_tmap_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, T, K, (uint64_t)K * 2, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -ERR_BAD_ARG;
  return dispatch(wfmt, BN, tmX, p, stream);
}

// As b200_gemm_wdec_gguf with split-K for small batches: `splits` CTAs share the K range of an output tile, leave fp32
// partials in `scratch` (splits * T * N floats) and the last one to arrive (tile_counters: one zeroed int per output
// tile, left zeroed) adds them up and writes bf16 (+ residual).  A decode-sized GEMM has too few 128-row tiles to
// occupy the GPU otherwise (8 at N = 1024).
extern "C" int b200_gemm_wdec_gguf_splitk(int wfmt, const void* W, const void* lut, const void* X, void* out_bf16,
                                          float* scratch, const void* residual, int T, int N, int K, int splits,
                                          int* tile_counters, int* status, cudaStream_t stream) {
  GemmParams p;
  if (!fill(p, wfmt, W, lut, out_bf16, scratch, residual, T, N, K, status) || !out_bf16 || splits < 1) return -ERR_BAD_ARG;
  if (splits > p.kb_total) splits = p.kb_total;
  {
    const int per = (p.kb_total + splits - 1) / splits;      // no split may end up with an empty K range
    splits = (p.kb_total + per - 1) / per;
  }
  if (splits > 1 && (!scratch || !tile_counters)) return -ERR_BAD_ARG;
  p.splits = splits;
  p.tile_counters = tile_counters;
  if (splits == 1) p.out_f32 = nullptr;
  int BN = T <= 16 ? 16 : T <= 32 ? 32 : T <= 64 ? 64 : T <= 128 ? 128 : 256;
  if (BN == 256 && !bn256_ok(wfmt)) BN = 128;
  p.n_tiles = (T + BN - 1) / BN;
  CUtensorMap tmX;
  if (!make_tmap_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, T, K, (uint64_t)K * 2, BN, BK, CU_TENSOR_MAP_SWIZZLE_128B))
    return -ERR_BAD_ARG;
  return dispatch(wfmt, BN, tmX, p, stream);
}

// Grouped form over expert-sorted rows (see b200_gemm_wdec_grouped): `groups` packed matrices back to back.
extern "C" int b200_gemm_wdec_gguf_grouped(int wfmt, const void* W, const void* lut, const void* X, void* out_bf16,
                                           int rows_total, int N, int K, int groups, const void* work_table,
                                           const int* num_work, int bn, int* status, cudaStream_t stream) {
  GemmParams p;
  if (!fill(p, wfmt, W, lut, out_bf16, nullptr, nullptr, rows_total, N, K, status) || !out_bf16 || !work_table || !num_work ||
      groups <= 0)
    return -ERR_BAD_ARG;
  p.work_table = reinterpret_cast<const int4*>(work_table);
  p.num_work = num_work;
  p.w_group_stride = (size_t)p.m_tiles * p.kb_total * raw_stage_bytes(wfmt);
  CUtensorMap tmX;
  if (!make_tmap_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, rows_total, K, (uint64_t)K * 2, bn, BK,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return -ERR_BAD_ARG;
  return dispatch(wfmt, bn, tmX, p, stream);
}
