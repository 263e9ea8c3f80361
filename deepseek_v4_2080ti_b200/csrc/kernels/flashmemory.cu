// FlashMemory retriever for very long contexts: for one decode token, score every compressed key chunk of a scorer
// layer, combine the scorer layers, keep the best chunks and turn them into KV row indices; the KV rows of chunks
// that are not kept can then live in host memory (runtime/kv_swap.py).
//
//   q side   : hidden -> wq_a -> RMSNorm(gamma) -> wq_b -> [heads, 128]; bf16 rounding, interleaved-pair RoPE (YaRN
//              frequencies) on the last rope_dim dims, orthonormal Hadamard rotation (fp32)
//   weights  : fused_w = (weights_proj @ hidden) * 128^-1/2 * heads^-1/2
//   score[c] = sigmoid( sum_h relu(q_h . k_c) * fused_w[h] ),  k_c = E4M3 bytes * fp32 chunk scale, or float keys
//   ensemble : max or mean over scorer layers;  top-k: best `keep` chunks in descending score order
//
// Reference behaviour: cpp_engine/include/flashmemory_ops.hpp:7-137 and backends/cuda/kernels/flashmemory_ops.cu
// (rope_hadamard :88, score_chunks :130, score_float_keys :192, ensemble :233, topk :256, write_global_indices :308).
// There every weight is fp32 and each head's dot product is a serial loop of one thread; here weights are bf16, the
// matvecs are warp-per-row, and a warp scores a chunk with the query heads spread over its lanes.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int D = 128;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16(v)); }

// y[n] = sum_k W[n, k] * xn[k], xn = x (gamma == null) or x * rsqrt(mean(x^2) + eps) * gamma.  Warp per row.
__global__ void fm_matvec_kernel(const __nv_bfloat16* __restrict__ W, const float* __restrict__ x, const float* __restrict__ gamma,
                                 float eps, float out_scale, float* __restrict__ y, int N, int K) {
  __shared__ float red[8];
  __shared__ float inv_s;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float inv = 1.f;
  if (gamma) {
    float ss = 0.f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) ss += x[k] * x[k];
    ss = warp_sum(ss);
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    if (threadIdx.x == 0) {
      float t = 0.f;
      for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
      inv_s = rsqrtf(t / (float)K + eps);
    }
    __syncthreads();
    inv = inv_s;
  }
  const int n = blockIdx.x * (blockDim.x >> 5) + warp;
  if (n >= N) return;
  const __nv_bfloat16* row = W + (size_t)n * K;
  float acc = 0.f;
  for (int k = lane * 2; k < K; k += 64) {
    const float2 w2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(row + k));
    const float x0 = gamma ? x[k] * inv * gamma[k] : x[k], x1 = gamma ? x[k + 1] * inv * gamma[k + 1] : x[k + 1];
    acc += w2.x * x0 + w2.y * x1;
  }
  acc = warp_sum(acc);
  if (lane == 0) y[n] = acc * out_scale;
}

// q [heads, 128] in place: round to bf16, rotate the last rope_dim dims (pairs (2i, 2i + 1)), Hadamard.  Warp per head.
__global__ void fm_rope_hadamard_kernel(float* __restrict__ q, const float* __restrict__ inv_freqs, int heads, int rope_dim,
                                        long long position) {
  const int head = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (head >= heads) return;
  const int lane = threadIdx.x & 31;
  float* row = q + (size_t)head * D + lane * 4;
  float v[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = round_bf16(row[i]);
  const int rope_start = D - rope_dim;
#pragma unroll
  for (int p = 0; p < 2; ++p) {
    const int d0 = lane * 4 + 2 * p;
    if (d0 >= rope_start) {
      const float ang = (float)position * inv_freqs[(d0 - rope_start) >> 1];
      float sn, cs;
      sincosf(ang, &sn, &cs);
      const float a = v[2 * p], b = v[2 * p + 1];
      v[2 * p] = round_bf16(a * cs - b * sn);
      v[2 * p + 1] = round_bf16(a * sn + b * cs);
    }
  }
  float t0 = v[0] + v[1], t1 = v[0] - v[1], t2 = v[2] + v[3], t3 = v[2] - v[3];
  v[0] = t0 + t2; v[1] = t1 + t3; v[2] = t0 - t2; v[3] = t1 - t3;
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? o - v[i] : v[i] + o;
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) row[i] = v[i] * 0.08838834764831845f;
}

// One warp per chunk; the query heads are spread over the lanes (head h on lane h % 32), the chunk's key is staged in
// shared memory once per warp.  q rows are padded to 129 floats so that lanes reading different heads hit different
// banks.
__global__ void __launch_bounds__(256)
fm_score_kernel(const float* __restrict__ q, const float* __restrict__ fused_w, const uint8_t* __restrict__ keys8,
                const float* __restrict__ keysf, float* __restrict__ scores, int n_chunks, int heads, int apply_sigmoid) {
  extern __shared__ float sm[];
  float* sq = sm;                                  // [heads][129]
  float* sk = sm + (size_t)heads * 129;            // [8 warps][128]
  for (int i = threadIdx.x; i < heads * D; i += blockDim.x) sq[(i >> 7) * 129 + (i & 127)] = q[i];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float* k = sk + warp * D;
  for (int c = blockIdx.x * 8 + warp; c < n_chunks; c += gridDim.x * 8) {
    if (keys8) {
      const uint8_t* row = keys8 + (size_t)c * (D + 4);
      const uint32_t w = *reinterpret_cast<const uint32_t*>(row + lane * 4);
      const float scale = __uint_as_float(*reinterpret_cast<const uint32_t*>(row + D));
      const __half2_raw r0 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xFFFF), __NV_E4M3);
      const __half2_raw r1 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r0));
      const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&r1));
      k[lane * 4] = a.x * scale; k[lane * 4 + 1] = a.y * scale; k[lane * 4 + 2] = b.x * scale; k[lane * 4 + 3] = b.y * scale;
    } else {
      const float4 f = *reinterpret_cast<const float4*>(keysf + (size_t)c * D + lane * 4);
      k[lane * 4] = f.x; k[lane * 4 + 1] = f.y; k[lane * 4 + 2] = f.z; k[lane * 4 + 3] = f.w;
    }
    __syncwarp();
    float local = 0.f;
    for (int h = lane; h < heads; h += 32) {
      const float* qh = sq + h * 129;
      float dot = 0.f;
#pragma unroll 8
      for (int d = 0; d < D; ++d) dot += qh[d] * k[d];
      local += fmaxf(dot, 0.f) * fused_w[h];
    }
    local = warp_sum(local);
    if (lane == 0) scores[c] = apply_sigmoid ? 1.f / (1.f + __expf(-local)) : local;
    __syncwarp();
  }
}

__global__ void fm_ensemble_kernel(const float* __restrict__ layer_scores, int n_layers, int n_chunks, int stride, int use_max,
                                   float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= n_chunks) return;
  float acc = use_max ? -INFINITY : 0.f;
  for (int l = 0; l < n_layers; ++l) {
    const float v = layer_scores[(size_t)l * stride + c];
    acc = use_max ? fmaxf(acc, v) : acc + v;
  }
  out[c] = use_max ? acc : acc / (float)n_layers;
}

// Single block: `keep` rounds of a block-wide arg-max over the chunks not taken yet (bit mask in shared memory).
// Descending score order, ties to the lower index.
__global__ void __launch_bounds__(1024)
fm_topk_kernel(const float* __restrict__ scores, int n_chunks, int keep, int* __restrict__ out_idx, float* __restrict__ out_val) {
  extern __shared__ uint32_t taken[];               // [(n_chunks + 31) / 32]
  __shared__ float bv[32];
  __shared__ int bi[32];
  const int words = (n_chunks + 31) >> 5;
  for (int i = threadIdx.x; i < words; i += blockDim.x) taken[i] = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  for (int r = 0; r < keep; ++r) {
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int c = threadIdx.x; c < n_chunks; c += blockDim.x) {
      if ((taken[c >> 5] >> (c & 31)) & 1u) continue;
      const float v = scores[c];
      if (v > best || (v == best && c < idx) || idx == 0x7fffffff) { best = v; idx = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
    }
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
      best = lane < nwarp ? bv[lane] : -INFINITY;
      idx = lane < nwarp ? bi[lane] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) { best = ov; idx = oi; }
      }
      if (lane == 0) {
        out_idx[r] = idx == 0x7fffffff ? -1 : idx;
        if (out_val) out_val[r] = idx == 0x7fffffff ? -INFINITY : best;
        if (idx != 0x7fffffff) taken[idx >> 5] |= 1u << (idx & 31);
      }
    }
    __syncthreads();
  }
}

__global__ void fm_write_indices_kernel(const int* __restrict__ logical, int keep, int offset, int* __restrict__ out) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < keep) out[i] = logical[i] < 0 ? -1 : offset + logical[i];
}

}  // namespace

// Scores of one scorer layer for one decode token.  hidden fp32 [hidden_dim]; wq_a bf16 [q_lora, hidden_dim]; wq_b
// bf16 [heads * 128, q_lora]; q_norm fp32 [q_lora]; weights_proj bf16 [heads, hidden_dim]; inv_freqs fp32
// [rope_dim / 2]; exactly one of keys8 (uint8 [n_chunks, 132]: 128 E4M3 bytes + fp32 scale) and keysf (fp32
// [n_chunks, 128]); scratch: q [heads * 128], qlora [q_lora], fused_w [heads]; scores fp32 [n_chunks].
extern "C" int b200_fm_score_layer(const float* hidden, const void* wq_a, const void* wq_b, const float* q_norm,
                                   const void* weights_proj, const float* inv_freqs, const void* keys8, const float* keysf,
                                   float* q_scratch, float* qlora_scratch, float* fused_w, float* scores, int n_chunks,
                                   int heads, int q_lora, int hidden_dim, int rope_dim, float eps, long long position,
                                   int apply_sigmoid, cudaStream_t stream) {
  if (!hidden || !wq_a || !wq_b || !q_norm || !weights_proj || !inv_freqs || (!keys8) == (!keysf) || !q_scratch ||
      !qlora_scratch || !fused_w || !scores)
    return -6;
  if (n_chunks < 0 || heads <= 0 || heads > 256 || q_lora <= 0 || (q_lora & 1) || hidden_dim <= 0 || (hidden_dim & 1) ||
      rope_dim < 0 || rope_dim > D || (rope_dim & 3))
    return -6;
  if (n_chunks == 0) return 0;
  const auto* a = reinterpret_cast<const __nv_bfloat16*>(wq_a);
  const auto* b = reinterpret_cast<const __nv_bfloat16*>(wq_b);
  const auto* wp = reinterpret_cast<const __nv_bfloat16*>(weights_proj);
  fm_matvec_kernel<<<(q_lora + 7) / 8, 256, 0, stream>>>(a, hidden, nullptr, 0.f, 1.f, qlora_scratch, q_lora, hidden_dim);
  fm_matvec_kernel<<<(heads * D + 7) / 8, 256, 0, stream>>>(b, qlora_scratch, q_norm, eps, 1.f, q_scratch, heads * D, q_lora);
  fm_rope_hadamard_kernel<<<(heads + 7) / 8, 256, 0, stream>>>(q_scratch, inv_freqs, heads, rope_dim, position);
  const float wscale = rsqrtf((float)D) * rsqrtf((float)heads);
  fm_matvec_kernel<<<(heads + 7) / 8, 256, 0, stream>>>(wp, hidden, nullptr, 0.f, wscale, fused_w, heads, hidden_dim);
  const size_t smem = ((size_t)heads * 129 + 8 * D) * sizeof(float);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(fm_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (256 * 129 + 8 * D) * (int)sizeof(float));
    attr_set = true;
  }
  const int blocks = min((n_chunks + 7) / 8, 148 * 4);
  fm_score_kernel<<<blocks, 256, smem, stream>>>(q_scratch, fused_w, reinterpret_cast<const uint8_t*>(keys8), keysf, scores,
                                                 n_chunks, heads, apply_sigmoid);
  return (int)cudaGetLastError();
}

extern "C" int b200_fm_ensemble(const float* layer_scores, int n_layers, int n_chunks, int stride, int use_max, float* out,
                                cudaStream_t stream) {
  if (!layer_scores || !out || n_layers <= 0 || n_chunks < 0 || stride < n_chunks) return -6;
  if (n_chunks == 0) return 0;
  fm_ensemble_kernel<<<(n_chunks + 255) / 256, 256, 0, stream>>>(layer_scores, n_layers, n_chunks, stride, use_max, out);
  return (int)cudaGetLastError();
}

// out_idx [keep]: chunk ids by descending score (-1 past n_chunks); out_val optional.  n_chunks <= 2^20.
extern "C" int b200_fm_topk(const float* scores, int n_chunks, int keep, int* out_idx, float* out_val, cudaStream_t stream) {
  if (!scores || !out_idx || n_chunks < 0 || keep < 0 || n_chunks > (1 << 20)) return -6;
  if (keep == 0) return 0;
  const size_t smem = (size_t)((n_chunks + 31) / 32 + 1) * sizeof(uint32_t);
  static bool attr_set = false;
  if (!attr_set) {
    cudaFuncSetAttribute(fm_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ((1 << 20) / 32 + 1) * (int)sizeof(uint32_t));
    attr_set = true;
  }
  fm_topk_kernel<<<1, 1024, smem, stream>>>(scores, n_chunks, keep, out_idx, out_val);
  return (int)cudaGetLastError();
}

extern "C" int b200_fm_write_global_indices(const int* logical, int keep, int offset, int* out, cudaStream_t stream) {
  if (!logical || !out || keep < 0) return -6;
  if (keep == 0) return 0;
  fm_write_indices_kernel<<<(keep + 255) / 256, 256, 0, stream>>>(logical, keep, offset, out);
  return (int)cudaGetLastError();
}
