// Quantised paged KV cache with one fp32 scale per (token, kv head) - fmt 1: FP8 E4M3 keys and values, fmt 2: INT8 keys
// and values, fmt 3 ("K8V4"): E4M3 keys and 4-bit affine values (scale + minimum per row, two values per byte, even
// dimension in the low nibble, rows of 64 bytes) - : quantising append from a bf16 staging cache,
// and the dequantisation of a sequence's cached range back into a bf16 staging cache for the tensor-core prefill
// kernel (which then sees exact bf16 rows for the current chunk and dequantised rows for the past).  The decode
// attention kernel reads the 8-bit rows directly (attn_gqa_decode.cu, b200_gqa_decode_kv8).
//
// Layouts: caches [num_blocks, Hkv, bs, 128] (one byte per element, or bf16), scales [num_blocks, Hkv, bs] fp32; a row's slot is
// block * bs + offset.  One warp per (token, head, K|V); lane l owns dims [4l, 4l + 4).
//
// Reference behaviour: the fp8, int8_per_token_head and turboquant_k8v4 KV-cache modes of the Qwen engine
// (cpp_engine/include/qwen_engine.hpp:14-29, qwen_fp8_ops.cu dequant_fp8_kv_cache :1203,
// qwen_int8_per_token_head_ops.cu append :16 / dequant :99 / decode attention :135, qwen_turboquant_ops.cu append :36
// (unscaled E5M2 keys there; scaled E4M3 here) / dequant :192); there the fp8 cache is
// dequantised for every attention call, here only the prefill path stages it.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int D = 128;
constexpr float E4M3_MAX = 448.f, INT8_MAX_F = 127.f;

__global__ void kv8_quantize_kernel(const __nv_bfloat16* __restrict__ stage_k, const __nv_bfloat16* __restrict__ stage_v,
                                       const int* __restrict__ src_slots, const int* __restrict__ dst_slots,
                                       uint8_t* __restrict__ k8, uint8_t* __restrict__ v8, float* __restrict__ k_scale,
                                       float* __restrict__ v_scale, float* __restrict__ v_min, int bs_src, int bs_dst, int T,
                                       int Hkv, int fmt) {
  const int lane = threadIdx.x & 31;
  const size_t w = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (size_t)T * Hkv * 2) return;
  const int which = (int)(w % 2), h = (int)((w / 2) % Hkv), t = (int)(w / (2 * Hkv));
  const int src = src_slots[t], dst = dst_slots[t];
  if (src < 0 || dst < 0) return;
  const __nv_bfloat16* sp = (which ? stage_v : stage_k) + (((size_t)(src / bs_src) * Hkv + h) * bs_src + src % bs_src) * D + lane * 4;
  const uint2 u = *reinterpret_cast<const uint2*>(sp);
  const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
  const float2 a = __bfloat1622float2(h2[0]), b = __bfloat1622float2(h2[1]);
  const size_t row = ((size_t)(dst / bs_dst) * Hkv + h) * bs_dst + dst % bs_dst;
  if (fmt == 3 && which) {
    float lo = fminf(fminf(a.x, a.y), fminf(b.x, b.y)), hi = fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, o));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, o));
    }
    const float scale = fmaxf((hi - lo) / 15.f, 1e-8f), inv = 1.f / scale;
    const int q0 = min(15, max(0, __float2int_rn((a.x - lo) * inv))), q1 = min(15, max(0, __float2int_rn((a.y - lo) * inv)));
    const int q2 = min(15, max(0, __float2int_rn((b.x - lo) * inv))), q3 = min(15, max(0, __float2int_rn((b.y - lo) * inv)));
    *reinterpret_cast<uint16_t*>(v8 + row * (D / 2) + lane * 2) = (uint16_t)(q0 | (q1 << 4) | (q2 << 8) | (q3 << 12));
    if (lane == 0) { v_scale[row] = scale; v_min[row] = lo; }
    return;
  }
  float amax = fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y)));
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float scale = fmaxf(amax, 1e-12f) / (fmt == 2 ? INT8_MAX_F : E4M3_MAX), inv = 1.f / scale;
  uint32_t packed;
  if (fmt == 2) {
    const int q0 = __float2int_rn(a.x * inv), q1 = __float2int_rn(a.y * inv), q2 = __float2int_rn(b.x * inv),
              q3 = __float2int_rn(b.y * inv);
    packed = (uint32_t)(q0 & 0xFF) | ((uint32_t)(q1 & 0xFF) << 8) | ((uint32_t)(q2 & 0xFF) << 16) | ((uint32_t)(q3 & 0xFF) << 24);
  } else {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a.x * inv, a.y * inv), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(b.x * inv, b.y * inv), __NV_SATFINITE, __NV_E4M3);
    packed = (uint32_t)lo | ((uint32_t)hi << 16);
  }
  *reinterpret_cast<uint32_t*>((which ? v8 : k8) + row * D + lane * 4) = packed;
  if (lane == 0) (which ? v_scale : k_scale)[row] = scale;
}

__global__ void kv8_dequantize_kernel(const uint8_t* __restrict__ k8, const uint8_t* __restrict__ v8,
                                         const float* __restrict__ k_scale, const float* __restrict__ v_scale,
                                         const float* __restrict__ v_min, const int* __restrict__ block_table, __nv_bfloat16* __restrict__ stage_k,
                                         __nv_bfloat16* __restrict__ stage_v, int bs, int n_tokens, int Hkv, int fmt) {
  const int lane = threadIdx.x & 31;
  const size_t w = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (w >= (size_t)n_tokens * Hkv * 2) return;
  const int which = (int)(w % 2), h = (int)((w / 2) % Hkv), j = (int)(w / (2 * Hkv));
  const int blk = block_table[j / bs];
  const size_t src = ((size_t)blk * Hkv + h) * bs + j % bs;
  const size_t dst = ((size_t)(j / bs) * Hkv + h) * bs + j % bs;          // staging keeps the sequence's own order
  const float s = (which ? v_scale : k_scale)[src];
  float2 a, b;                                              // dequantised values
  if (fmt == 3 && which) {
    const uint32_t n4 = *reinterpret_cast<const uint16_t*>(v8 + src * (D / 2) + lane * 2);
    const float m = v_min[src];
    a = make_float2((float)(n4 & 15) * s + m, (float)((n4 >> 4) & 15) * s + m);
    b = make_float2((float)((n4 >> 8) & 15) * s + m, (float)(n4 >> 12) * s + m);
  } else {
    const uint32_t q = *reinterpret_cast<const uint32_t*>((which ? v8 : k8) + src * D + lane * 4);
    if (fmt == 2) {
      a = make_float2((float)(int8_t)(q & 0xFF), (float)(int8_t)((q >> 8) & 0xFF));
      b = make_float2((float)(int8_t)((q >> 16) & 0xFF), (float)(int8_t)(q >> 24));
    } else {
      const __half2_raw r0 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(q & 0xFFFF), __NV_E4M3);
      const __half2_raw r1 = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(q >> 16), __NV_E4M3);
      a = __half22float2(*reinterpret_cast<const __half2*>(&r0));
      b = __half22float2(*reinterpret_cast<const __half2*>(&r1));
    }
    a.x *= s; a.y *= s; b.x *= s; b.y *= s;
  }
  const __nv_bfloat162 o0 = __floats2bfloat162_rn(a.x, a.y), o1 = __floats2bfloat162_rn(b.x, b.y);
  uint2 u;
  u.x = *reinterpret_cast<const uint32_t*>(&o0);
  u.y = *reinterpret_cast<const uint32_t*>(&o1);
  *reinterpret_cast<uint2*>((which ? stage_v : stage_k) + dst * D + lane * 4) = u;
}

}  // namespace

// Quantise T staged rows (slot src_slots[t] of the bf16 staging caches, block size bs_src) into slot dst_slots[t] of
// the quantised caches (block size bs_dst; fmt 1 = E4M3, 2 = INT8, 3 = E4M3 keys + 4-bit values); negative slots are
// skipped.
extern "C" int b200_kv8_quantize(const void* stage_k, const void* stage_v, const int* src_slots, const int* dst_slots,
                                 void* k8, void* v8, float* k_scale, float* v_scale, float* v_min, int bs_src, int bs_dst,
                                 int T, int Hkv, int fmt, cudaStream_t stream) {
  if (T <= 0 || Hkv <= 0 || bs_src <= 0 || bs_dst <= 0 || fmt < 1 || fmt > 3 || (fmt == 3 && !v_min)) return -6;
  const size_t warps = (size_t)T * Hkv * 2;
  kv8_quantize_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(stage_k), reinterpret_cast<const __nv_bfloat16*>(stage_v), src_slots, dst_slots,
      reinterpret_cast<uint8_t*>(k8), reinterpret_cast<uint8_t*>(v8), k_scale, v_scale, v_min, bs_src, bs_dst, T, Hkv, fmt);
  return (int)cudaGetLastError();
}

// Dequantise the first n_tokens positions of one sequence (its block-table row) into bf16 staging caches laid out as
// consecutive blocks 0, 1, 2, ... of the same block size.
extern "C" int b200_kv8_dequantize(const void* k8, const void* v8, const float* k_scale, const float* v_scale,
                                   const float* v_min, const int* block_table_row, void* stage_k, void* stage_v, int bs,
                                   int n_tokens, int Hkv, int fmt, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (Hkv <= 0 || bs <= 0 || fmt < 1 || fmt > 3 || (fmt == 3 && !v_min)) return -6;
  const size_t warps = (size_t)n_tokens * Hkv * 2;
  kv8_dequantize_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(k8), reinterpret_cast<const uint8_t*>(v8), k_scale, v_scale, v_min, block_table_row,
      reinterpret_cast<__nv_bfloat16*>(stage_k), reinterpret_cast<__nv_bfloat16*>(stage_v), bs, n_tokens, Hkv, fmt);
  return (int)cudaGetLastError();
}
