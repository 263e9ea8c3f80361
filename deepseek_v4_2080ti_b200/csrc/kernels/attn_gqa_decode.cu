// Paged GQA decode attention (one new query row per sequence), split over the
// context, head_dim 128.  Bandwidth-bound: each CTA streams a contiguous key
// range of one KV head through 16-byte loads (half a warp per key row) and
// serves all G query heads that share it, keeping online-softmax state in
// registers; partial (max, sum, O) states are merged in shared memory and,
// across context splits, by a small merge kernel.  Optional sigmoid output gate.
//
// Reference behaviour: cpp_engine/backends/cuda/kernels/qwen_gqa_optimized.cu
// (gqa_decode_split_f16 :1648, gqa_decode_merge_f16 :2457) and the paged KV
// gather of qwen_half_ops.cu:2798 (here the kernel reads the block table itself).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "ops.h"
#include "launch.h"

namespace {

constexpr int D = 128;
constexpr int THREADS = 128;
constexpr int NSTATE = 8;  // 4 warps x 2 half-warps

struct DecodeParams {
  const __nv_bfloat16* q;        // [B, Hq, D]
  const __nv_bfloat16* k_cache;  // [num_blocks, Hkv, bs, D]
  const __nv_bfloat16* v_cache;
  const int* block_table;        // [B, max_blocks]
  const int* kv_len;             // [B]
  float* partial;                // [B, Hq, splits, D + 2]
  __nv_bfloat16* out;            // [B, Hq, D]
  const __nv_bfloat16* gate;     // optional [B, Hq, D]
  int max_blocks, bs, Hq, Hkv, splits;
  float scale_log2;
  int window, sinks;             // window > 0: only the first `sinks` and the last `window` keys are visible
  // KV 1 / 2: the caches hold E4M3 / INT8 bytes (same [num_blocks, Hkv, bs, D] layout) with one fp32 scale per
  // (block, head, row); KV 3: E4M3 keys, 4-bit affine values (rows of D / 2 bytes, scale and minimum per row)
  const float* k_scale;
  const float* v_scale;
  const float* v_min;
};

__device__ __forceinline__ void e4m3x8_to_float(const uint2 u, float (&f)[8]) {
  const uint32_t w[2] = {u.x, u.y};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const __half2_raw r = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)((w[i >> 1] >> (16 * (i & 1))) & 0xFFFF), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&r));
    f[2 * i] = a.x;
    f[2 * i + 1] = a.y;
  }
}

__device__ __forceinline__ void int8x8_to_float(const uint2 u, float (&f)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = (float)(int8_t)(((i < 4 ? u.x : u.y) >> (8 * (i & 3))) & 0xFF);
}

template <int G, int KV>
__global__ void __launch_bounds__(THREADS)
gqa_decode_kernel(DecodeParams p) {
  __shared__ float s_m[NSTATE][G], s_l[NSTATE][G];
  __shared__ float s_o[NSTATE][G][D];
  b200::pdl_grid_trigger();
  b200::pdl_grid_wait();
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = lane >> 4, dl = lane & 15;
  const int kv_total = p.kv_len[b];
  // with a sliding window the visible keys are renumbered densely: [0, sinks) then the last `window` keys
  const bool windowed = p.window > 0 && kv_total > p.sinks + p.window;
  const int kv_len = windowed ? p.sinks + p.window : kv_total;
  const int win_shift = kv_total - p.window - p.sinks;          // dense index j >= sinks is key j + win_shift
  const int per = (kv_len + p.splits - 1) / p.splits;
  const int k0 = split * per, k1 = min(kv_len, k0 + per);
  const int* bt = p.block_table + (size_t)b * p.max_blocks;

  float q[G][8], acc[G][8], m[G], l[G];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const uint4 u = *reinterpret_cast<const uint4*>(p.q + ((size_t)b * p.Hq + kvh * G + g) * D + dl * 8);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(h2[i]);
      q[g][2 * i] = f.x * p.scale_log2;
      q[g][2 * i + 1] = f.y * p.scale_log2;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
    m[g] = -INFINITY;
    l[g] = 0.f;
  }

  for (int base = k0 + warp * 2; base < k1; base += 8) {
    // the loop bound is warp-uniform: every lane runs the shuffles, rows past the range contribute nothing
    const int kk = base + half;
    const bool valid = kk < k1;
    int kc = valid ? kk : k0;
    if (windowed && kc >= p.sinks) kc += win_shift;
    const int blk = bt[kc / p.bs];
    const size_t row = ((size_t)(blk * p.Hkv + kvh) * p.bs + (kc % p.bs)) * D + dl * 8;
    float kf[8], vf[8];
    float ks = 1.f;
    if constexpr (KV == 3) {
      const uint2 ku = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.k_cache) + row);
      const uint32_t vn = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const uint8_t*>(p.v_cache) + (row >> 1));
      ks = p.k_scale[row >> 7];
      const float vs = p.v_scale[row >> 7], vm = p.v_min[row >> 7];
      e4m3x8_to_float(ku, kf);
#pragma unroll
      for (int i = 0; i < 8; ++i) vf[i] = (float)((vn >> (4 * i)) & 15) * vs + vm;
    } else if constexpr (KV != 0) {
      const uint2 ku = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.k_cache) + row);
      const uint2 vu = *reinterpret_cast<const uint2*>(reinterpret_cast<const uint8_t*>(p.v_cache) + row);
      ks = p.k_scale[row >> 7];
      const float vs = p.v_scale[row >> 7];
      if constexpr (KV == 1) {
        e4m3x8_to_float(ku, kf);
        e4m3x8_to_float(vu, vf);
      } else {
        int8x8_to_float(ku, kf);
        int8x8_to_float(vu, vf);
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) vf[i] *= vs;
    } else {
      const uint4 ku = *reinterpret_cast<const uint4*>(p.k_cache + row);
      const uint4 vu = *reinterpret_cast<const uint4*>(p.v_cache + row);
      const __nv_bfloat162* kh = reinterpret_cast<const __nv_bfloat162*>(&ku);
      const __nv_bfloat162* vh = reinterpret_cast<const __nv_bfloat162*>(&vu);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 a = __bfloat1622float2(kh[i]);
        float2 c = __bfloat1622float2(vh[i]);
        kf[2 * i] = a.x; kf[2 * i + 1] = a.y;
        vf[2 * i] = c.x; vf[2 * i + 1] = c.y;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float s = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) s += q[g][i] * kf[i];
      s += __shfl_xor_sync(0xffffffffu, s, 8);
      s += __shfl_xor_sync(0xffffffffu, s, 4);
      s += __shfl_xor_sync(0xffffffffu, s, 2);
      s += __shfl_xor_sync(0xffffffffu, s, 1);
      if constexpr (KV != 0) s *= ks;
      if (valid) {
        const float mn = fmaxf(m[g], s);
        const float alpha = exp2f(m[g] - mn);
        const float pe = exp2f(s - mn);
        l[g] = l[g] * alpha + pe;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * alpha + pe * vf[i];
        m[g] = mn;
      }
    }
  }

  const int st = warp * 2 + half;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (dl == 0) { s_m[st][g] = m[g]; s_l[st][g] = l[g]; }
#pragma unroll
    for (int i = 0; i < 8; ++i) s_o[st][g][dl * 8 + i] = acc[g][i];
  }
  __syncthreads();
  const int d = threadIdx.x;  // one output dim per thread
#pragma unroll
  for (int g = 0; g < G; ++g) {
    float M = -INFINITY;
#pragma unroll
    for (int s = 0; s < NSTATE; ++s) M = fmaxf(M, s_m[s][g]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int s = 0; s < NSTATE; ++s) {
      const float w = (s_m[s][g] == -INFINITY) ? 0.f : exp2f(s_m[s][g] - M);
      L += s_l[s][g] * w;
      O += s_o[s][g][d] * w;
    }
    const int hq = kvh * G + g;
    if (p.splits == 1) {
      float o = L > 0.f ? O / L : 0.f;
      const size_t idx = ((size_t)b * p.Hq + hq) * D + d;
      if (p.gate) o *= 1.f / (1.f + __expf(-__bfloat162float(p.gate[idx])));
      p.out[idx] = __float2bfloat16(o);
    } else {
      float* dst = p.partial + (((size_t)b * p.Hq + hq) * p.splits + split) * (D + 2);
      dst[d] = O;
      if (d == 0) { dst[D] = M; dst[D + 1] = L; }
    }
  }
}

__global__ void gqa_decode_merge_kernel(const float* __restrict__ partial, int splits,
                                        const __nv_bfloat16* __restrict__ gate, __nv_bfloat16* __restrict__ out) {
  b200::pdl_grid_trigger();
  b200::pdl_grid_wait();
  const size_t bh = blockIdx.x;  // b * Hq + hq
  const int d = threadIdx.x;
  const float* base = partial + bh * splits * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, base[s * (D + 2) + D]);
  float L = 0.f, O = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = base[s * (D + 2) + D];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += base[s * (D + 2) + D + 1] * w;
    O += base[s * (D + 2) + d] * w;
  }
  float o = L > 0.f ? O / L : 0.f;
  const size_t idx = bh * D + d;
  if (gate) o *= 1.f / (1.f + __expf(-__bfloat162float(gate[idx])));
  out[idx] = __float2bfloat16(o);
}

}  // namespace

static thread_local int g_window = 0, g_sinks = 0;   // set by b200_gqa_decode_ex for the launch it wraps

// q/out/gate: [B, Hq, 128] bf16; caches [num_blocks, Hkv, block_size, 128]; workspace: fp32
// [B * Hq * splits * 130] (used when splits > 1).
static int decode_launch(int fmt, const void* q, const void* k_cache, const void* v_cache, const float* k_scale, const float* v_scale,
                         const float* v_min,
                         void* out, const void* gate, const int* block_table, const int* kv_len, float* workspace, int batch,
                         int max_blocks, int block_size, int n_q_heads, int n_kv_heads, int splits, float softmax_scale,
                         cudaStream_t stream) {
  if (n_q_heads % n_kv_heads || splits < 1) return -6;
  const int G = n_q_heads / n_kv_heads;
  DecodeParams p;
  p.q = reinterpret_cast<const __nv_bfloat16*>(q);
  p.k_cache = reinterpret_cast<const __nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<const __nv_bfloat16*>(v_cache);
  p.block_table = block_table;
  p.kv_len = kv_len;
  p.partial = workspace;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.gate = reinterpret_cast<const __nv_bfloat16*>(gate);
  p.max_blocks = max_blocks;
  p.bs = block_size;
  p.Hq = n_q_heads;
  p.Hkv = n_kv_heads;
  p.splits = splits;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.window = g_window;
  p.sinks = g_sinks;
  p.k_scale = k_scale;
  p.v_scale = v_scale;
  p.v_min = v_min;
  if (splits > 1 && !workspace) return -6;
  dim3 grid(splits, n_kv_heads, batch);
  cudaError_t e = cudaSuccess;
#define B200_DECODE_CASE(g)                                                                                   \
  case g:                                                                                                     \
    e = fmt == 1   ? b200::launch_pdl(gqa_decode_kernel<g, 1>, grid, dim3(THREADS), 0, stream, p)             \
        : fmt == 2 ? b200::launch_pdl(gqa_decode_kernel<g, 2>, grid, dim3(THREADS), 0, stream, p)             \
        : fmt == 3 ? b200::launch_pdl(gqa_decode_kernel<g, 3>, grid, dim3(THREADS), 0, stream, p)             \
                   : b200::launch_pdl(gqa_decode_kernel<g, 0>, grid, dim3(THREADS), 0, stream, p);            \
    break;
  switch (G) {
    B200_DECODE_CASE(1) B200_DECODE_CASE(2) B200_DECODE_CASE(3) B200_DECODE_CASE(4) B200_DECODE_CASE(5) B200_DECODE_CASE(6)
    B200_DECODE_CASE(8)
    default: return -6;
  }
#undef B200_DECODE_CASE
  if (e != cudaSuccess) return (int)e;
  if (splits > 1)
    e = b200::launch_pdl(gqa_decode_merge_kernel, dim3(batch * n_q_heads), dim3(D), 0, stream,
                         (const float*)workspace, splits, p.gate, p.out);
  return (int)e;
}

extern "C" int b200_gqa_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                               const void* gate, const int* block_table, const int* kv_len, float* workspace,
                               int batch, int max_blocks, int block_size, int n_q_heads, int n_kv_heads,
                               int splits, float softmax_scale, cudaStream_t stream) {
  return decode_launch(0, q, k_cache, v_cache, nullptr, nullptr, nullptr, out, gate, block_table, kv_len, workspace, batch, max_blocks,
                       block_size, n_q_heads, n_kv_heads, splits, softmax_scale, stream);
}

// Decode attention over a quantised cache (fmt 1 = E4M3, 2 = INT8, 3 = E4M3 keys + 4-bit affine values with v_min)
// with per-(token, head) fp32 scales [num_blocks, Hkv, bs]; the rows are dequantised in registers, so the kernel
// streams half (fmt 3: three eighths) of the bytes of the bf16 cache.  window / sinks as below.
extern "C" int b200_gqa_decode_kv8(int fmt, const void* q, const void* k8, const void* v8, const float* k_scale,
                                   const float* v_scale, const float* v_min, void* out, const void* gate, const int* block_table,
                                   const int* kv_len, float* workspace, int batch, int max_blocks, int block_size,
                                   int n_q_heads, int n_kv_heads, int splits, float softmax_scale, int window, int sinks,
                                   cudaStream_t stream) {
  if (!k_scale || !v_scale || fmt < 1 || fmt > 3 || (fmt == 3 && !v_min)) return -6;
  g_window = window > 0 ? window : 0;
  g_sinks = sinks > 0 ? sinks : 0;
  const int rc = decode_launch(fmt, q, k8, v8, k_scale, v_scale, v_min, out, gate, block_table, kv_len, workspace, batch, max_blocks,
                               block_size, n_q_heads, n_kv_heads, splits, softmax_scale, stream);
  g_window = g_sinks = 0;
  return rc;
}

// As b200_gqa_decode with a sliding window: each query sees the first `sinks` keys and the last `window` keys of its
// sequence (window <= 0: every key).
extern "C" int b200_gqa_decode_ex(const void* q, const void* k_cache, const void* v_cache, void* out, const void* gate,
                                  const int* block_table, const int* kv_len, float* workspace, int batch, int max_blocks,
                                  int block_size, int n_q_heads, int n_kv_heads, int splits, float softmax_scale, int window,
                                  int sinks, cudaStream_t stream) {
  g_window = window > 0 ? window : 0;
  g_sinks = sinks > 0 ? sinks : 0;
  const int rc = b200_gqa_decode(q, k_cache, v_cache, out, gate, block_table, kv_len, workspace, batch, max_blocks, block_size,
                                 n_q_heads, n_kv_heads, splits, softmax_scale, stream);
  g_window = g_sinks = 0;
  return rc;
}
