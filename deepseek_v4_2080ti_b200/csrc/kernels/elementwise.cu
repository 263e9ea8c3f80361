// Bandwidth-bound row kernels: RMSNorm family (plain, (1+gamma), fused residual
// add, gated), embedding gather, SwiGLU / sigmoid gating, causal depthwise
// conv + SiLU with a carried tail, Gated-DeltaNet gate math, split-K finishing
// fused with the residual add and the norm.  All activations are bf16, all
// arithmetic fp32, 16-byte vector accesses.
//
// Reference behaviour: cpp_engine/backends/cuda/kernels/qwen_half_ops.cu
// (rmsnorm :1883-2100, gated_rmsnorm :2101-2183, conv_silu :2198-2264,
// linear_gates :2265-2281, sigmoid_mul/silu_mul :2730-2745, embedding :1854).
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  v = warp_sum(v);
  if (lane == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

struct bf16x8 {
  uint4 u;
  __device__ __forceinline__ void unpack(float (&f)[8]) const {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 t = __bfloat1622float2(h[i]);
      f[2 * i] = t.x;
      f[2 * i + 1] = t.y;
    }
  }
  __device__ __forceinline__ void pack(const float (&f)[8]) {
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  }
};

// One block per row. Optional: residual add (x += delta, written back), fp32 split-K
// partials summed into the residual first, unit offset on gamma.
// cols % 8 == 0. Row is cached in registers for cols <= 8 * 8 * blockDim.
template <int MAX_VEC>
__global__ void rmsnorm_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                               const float* __restrict__ partials, int splits, size_t split_stride,
                               const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ out,
                               int cols, float eps, int unit_offset, int write_x) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const int nvec = cols >> 3;
  float cache[MAX_VEC][8];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < MAX_VEC; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      bf16x8 a;
      a.u = *reinterpret_cast<const uint4*>(x + row * cols + v * 8);
      a.unpack(cache[it]);
      if (delta) {
        bf16x8 d;
        d.u = *reinterpret_cast<const uint4*>(delta + row * cols + v * 8);
        float df[8];
        d.unpack(df);
#pragma unroll
        for (int j = 0; j < 8; ++j) cache[it][j] += df[j];
      }
      if (partials) {
        for (int s = 0; s < splits; ++s) {
          const float4* p = reinterpret_cast<const float4*>(partials + s * split_stride + row * cols + v * 8);
          float4 p0 = p[0], p1 = p[1];
          cache[it][0] += p0.x; cache[it][1] += p0.y; cache[it][2] += p0.z; cache[it][3] += p0.w;
          cache[it][4] += p1.x; cache[it][5] += p1.y; cache[it][6] += p1.z; cache[it][7] += p1.w;
        }
      }
      if (delta || partials) {
        // the residual stream is bf16: round first so norm input == stored residual
        bf16x8 r;
        r.pack(cache[it]);
        if (write_x) *reinterpret_cast<uint4*>(x + row * cols + v * 8) = r.u;
        r.unpack(cache[it]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += cache[it][j] * cache[it][j];
    }
  }
  const float inv = rsqrtf(block_sum(ss, red) / (float)cols + eps);
  if (!out) return;
#pragma unroll
  for (int it = 0; it < MAX_VEC; ++it) {
    const int v = threadIdx.x + it * blockDim.x;
    if (v < nvec) {
      bf16x8 g;
      g.u = *reinterpret_cast<const uint4*>(gamma + v * 8);
      float gf[8], o[8];
      g.unpack(gf);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = cache[it][j] * inv * (unit_offset ? 1.f + gf[j] : gf[j]);
      bf16x8 r;
      r.pack(o);
      *reinterpret_cast<uint4*>(out + row * cols + v * 8) = r.u;
    }
  }
}

// Per-head norm over head_dim (<= 256, % 8 == 0) with a SiLU gate: one warp per (row, head).
__global__ void gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                                     const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ out,
                                     size_t nrows, int dim, float eps, int heads, size_t gate_ld) {
  const size_t row = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= nrows) return;
  const int lane = threadIdx.x & 31;
  const int v = lane;  // one 8-wide vector per lane (dim <= 256)
  float xf[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const bool act = v * 8 < dim;
  if (act) {
    bf16x8 a;
    a.u = *reinterpret_cast<const uint4*>(x + row * dim + v * 8);
    a.unpack(xf);
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += xf[j] * xf[j];
  const float inv = rsqrtf(warp_sum(ss) / (float)dim + eps);
  if (act) {
    bf16x8 g, z;
    g.u = *reinterpret_cast<const uint4*>(gamma + v * 8);
    // gate row (t, head) may live inside a wider projection output: gate + t * gate_ld + head * dim
    z.u = *reinterpret_cast<const uint4*>(gate + (row / heads) * gate_ld + (row % heads) * dim + v * 8);
    float gf[8], zf[8], o[8];
    g.unpack(gf);
    z.unpack(zf);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = xf[j] * inv * gf[j] * silu_f(zf[j]);
    bf16x8 r;
    r.pack(o);
    *reinterpret_cast<uint4*>(out + row * dim + v * 8) = r.u;
  }
}

__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int hidden, int vocab_lo, int vocab_hi) {
  const size_t row = blockIdx.x;
  const int id = ids[row];
  const bool in = id >= vocab_lo && id < vocab_hi;
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)(in ? id - vocab_lo : 0) * hidden);
  uint4* dst = reinterpret_cast<uint4*>(out + row * hidden);
  for (int v = threadIdx.x; v < (hidden >> 3); v += blockDim.x) dst[v] = in ? src[v] : make_uint4(0, 0, 0, 0);
}

// out[t, i] = silu(gu[t, i]) * gu[t, inter + i]   (gate and up come from one fused GEMM)
__global__ void silu_mul_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ out,
                                size_t rows, int inter) {
  const size_t nvec = rows * (size_t)(inter >> 3);
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
    const size_t r = i / (inter >> 3);
    const int v = (int)(i % (inter >> 3));
    bf16x8 g, u;
    g.u = *reinterpret_cast<const uint4*>(gu + r * 2 * inter + v * 8);
    u.u = *reinterpret_cast<const uint4*>(gu + r * 2 * inter + inter + v * 8);
    float gf[8], uf[8], o[8];
    g.unpack(gf);
    u.unpack(uf);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = silu_f(gf[j]) * uf[j];
    bf16x8 rr;
    rr.pack(o);
    *reinterpret_cast<uint4*>(out + r * inter + v * 8) = rr.u;
  }
}

__global__ void sigmoid_mul_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ gate,
                                   __nv_bfloat16* __restrict__ out, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    bf16x8 a, g;
    a.u = reinterpret_cast<const uint4*>(x)[i];
    g.u = reinterpret_cast<const uint4*>(gate)[i];
    float af[8], gf[8], o[8];
    a.unpack(af);
    g.unpack(gf);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = af[j] * sigmoid_f(gf[j]);
    bf16x8 r;
    r.pack(o);
    reinterpret_cast<uint4*>(out)[i] = r.u;
  }
}

__global__ void add_kernel(__nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ x, size_t n8) {
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
    bf16x8 a, b;
    a.u = reinterpret_cast<const uint4*>(y)[i];
    b.u = reinterpret_cast<const uint4*>(x)[i];
    float af[8], bf[8];
    a.unpack(af);
    b.unpack(bf);
#pragma unroll
    for (int j = 0; j < 8; ++j) af[j] += bf[j];
    a.pack(af);
    reinterpret_cast<uint4*>(y)[i] = a.u;
  }
}

// Causal depthwise conv (kernel KW <= 4) + SiLU over a token-major [T, C] tensor.
// tail: [KW-1, C] = the last KW-1 inputs of the previous chunk (zeros at sequence start);
// updated in place when update_tail. Thread = 8 channels, grid.y tiles time.
template <int KW>
__global__ void conv_silu_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                                 __nv_bfloat16* __restrict__ tail, __nv_bfloat16* __restrict__ y, int ldy,
                                 int T, int C, int t_per_block, int update_tail) {
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int t_begin = blockIdx.y * t_per_block;
  const int t_end = min(T, t_begin + t_per_block);
  float wf[8][KW];
#pragma unroll
  for (int j = 0; j < 8; ++j)
#pragma unroll
    for (int k = 0; k < KW; ++k) wf[j][k] = __bfloat162float(w[(size_t)(c0 + j) * KW + k]);
  float hist[KW - 1][8];
#pragma unroll
  for (int k = 0; k < KW - 1; ++k) {
    const int ts = t_begin - (KW - 1) + k;
    bf16x8 a;
    if (ts >= 0) a.u = *reinterpret_cast<const uint4*>(x + (size_t)ts * ldx + c0);
    else a.u = *reinterpret_cast<const uint4*>(tail + (size_t)(ts + KW - 1) * C + c0);
    a.unpack(hist[k]);
  }
  for (int t = t_begin; t < t_end; ++t) {
    bf16x8 a;
    a.u = *reinterpret_cast<const uint4*>(x + (size_t)t * ldx + c0);
    float cur[8], o[8];
    a.unpack(cur);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float acc = cur[j] * wf[j][KW - 1];
#pragma unroll
      for (int k = 0; k < KW - 1; ++k) acc += hist[k][j] * wf[j][k];
      o[j] = silu_f(acc);
    }
    bf16x8 r;
    r.pack(o);
    *reinterpret_cast<uint4*>(y + (size_t)t * ldy + c0) = r.u;
#pragma unroll
    for (int k = 0; k + 1 < KW - 1; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) hist[k][j] = hist[k + 1][j];
#pragma unroll
    for (int j = 0; j < 8; ++j) hist[KW - 2][j] = cur[j];
  }
  // Only the block that owns the end of the chunk rewrites the tail, and only after
  // every block has read the old one: the caller launches tail updates separately
  // when gridDim.y > 1 (see b200_conv_silu).
  if (update_tail && t_end == T && gridDim.y == 1) {
#pragma unroll
    for (int k = 0; k < KW - 1; ++k) {
      bf16x8 r;
      r.pack(hist[k]);
      *reinterpret_cast<uint4*>(tail + (size_t)k * C + c0) = r.u;
    }
  }
}

// New tail = last KW-1 rows of [old tail ; x].
__global__ void conv_tail_update_kernel(const __nv_bfloat16* __restrict__ x, int ldx,
                                        __nv_bfloat16* __restrict__ tail, int T, int C, int KW) {
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  uint4 rows[3];
  for (int k = 0; k < KW - 1; ++k) {
    const int ts = T - (KW - 1) + k;
    rows[k] = ts >= 0 ? *reinterpret_cast<const uint4*>(x + (size_t)ts * ldx + c0)
                      : *reinterpret_cast<const uint4*>(tail + (size_t)(ts + KW - 1) * C + c0);
  }
  for (int k = 0; k < KW - 1; ++k) *reinterpret_cast<uint4*>(tail + (size_t)k * C + c0) = rows[k];
}

// Batched single-token conv: row b uses tail slot slot_ids[b] (or b).
template <int KW>
__global__ void conv_silu_step_kernel(const __nv_bfloat16* __restrict__ x, int ldx, const __nv_bfloat16* __restrict__ w,
                                      __nv_bfloat16* __restrict__ tails, size_t slot_stride,
                                      const int* __restrict__ slot_ids, __nv_bfloat16* __restrict__ y, int ldy, int C) {
  const int c0 = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c0 >= C) return;
  const int b = blockIdx.y;
  __nv_bfloat16* tail = tails + (size_t)(slot_ids ? slot_ids[b] : b) * slot_stride;
  bf16x8 a;
  a.u = *reinterpret_cast<const uint4*>(x + (size_t)b * ldx + c0);
  float cur[8], o[8], h[KW - 1][8];
  a.unpack(cur);
#pragma unroll
  for (int k = 0; k < KW - 1; ++k) {
    bf16x8 t;
    t.u = *reinterpret_cast<const uint4*>(tail + (size_t)k * C + c0);
    t.unpack(h[k]);
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    float acc = cur[j] * __bfloat162float(w[(size_t)(c0 + j) * KW + KW - 1]);
#pragma unroll
    for (int k = 0; k < KW - 1; ++k) acc += h[k][j] * __bfloat162float(w[(size_t)(c0 + j) * KW + k]);
    o[j] = silu_f(acc);
  }
  bf16x8 r;
  r.pack(o);
  *reinterpret_cast<uint4*>(y + (size_t)b * ldy + c0) = r.u;
#pragma unroll
  for (int k = 0; k + 1 < KW - 1; ++k) {
    bf16x8 t;
    t.pack(h[k + 1]);
    *reinterpret_cast<uint4*>(tail + (size_t)k * C + c0) = t.u;
  }
  *reinterpret_cast<uint4*>(tail + (size_t)(KW - 2) * C + c0) = a.u;
}

// g = -exp(A_log) * softplus(a + dt_bias)  (log-decay), beta = sigmoid(b); fp32 outputs.
__global__ void gdn_gates_kernel(const __nv_bfloat16* __restrict__ ab, int ld, int a_off, int b_off,
                                 const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                                 float* __restrict__ g, float* __restrict__ beta, size_t rows, int heads) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * heads) return;
  const size_t r = i / heads;
  const int h = (int)(i % heads);
  const float av = __bfloat162float(ab[r * ld + a_off + h]) + dt_bias[h];
  const float sp = av > 20.f ? av : log1pf(expf(av));
  g[i] = -expf(a_log[h]) * sp;
  beta[i] = sigmoid_f(__bfloat162float(ab[r * ld + b_off + h]));
}

// Row arg-max over fp32 or bf16 logits; writes (index + index_offset) and value. One block per row.
template <typename T>
__global__ void argmax_kernel(const T* __restrict__ logits, int ld, int n, int index_offset,
                              int* __restrict__ out_idx, float* __restrict__ out_val) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const T* row = logits + (size_t)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = (float)row[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int nw = blockDim.x >> 5;
    best = threadIdx.x < nw ? sv[threadIdx.x] : -INFINITY;
    bi = threadIdx.x < nw ? si[threadIdx.x] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (threadIdx.x == 0) {
      out_idx[blockIdx.x] = bi + index_offset;
      if (out_val) out_val[blockIdx.x] = best;
    }
  }
}

// Two-stage variant for few rows over a wide vocabulary: grid (chunks, rows) writes one (value, index) pair
// per chunk, a second small launch reduces the pairs.  A single block per row would leave 147 SMs idle.
constexpr int kArgmaxChunks = 64;
constexpr int kArgmaxMaxRows = 64;
__device__ float g_argmax_val[kArgmaxMaxRows * kArgmaxChunks];
__device__ int g_argmax_idx[kArgmaxMaxRows * kArgmaxChunks];

template <typename T>
__global__ void argmax_chunk_kernel(const T* __restrict__ logits, int ld, int n, int chunk) {
  __shared__ float sv[8];
  __shared__ int si[8];
  const T* row = logits + (size_t)blockIdx.y * ld;
  const int lo = blockIdx.x * chunk, hi = min(n, lo + chunk);
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    const float v = (float)row[i];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
      if (sv[w] > best || (sv[w] == best && si[w] < bi)) { best = sv[w]; bi = si[w]; }
    g_argmax_val[blockIdx.y * kArgmaxChunks + blockIdx.x] = best;
    g_argmax_idx[blockIdx.y * kArgmaxChunks + blockIdx.x] = bi;
  }
}

__global__ void argmax_final_kernel(int chunks, int index_offset, int* __restrict__ out_idx,
                                    float* __restrict__ out_val) {
  const int r = blockIdx.x, lane = threadIdx.x;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < chunks; c += 32) {
    const float v = g_argmax_val[r * kArgmaxChunks + c];
    const int i = g_argmax_idx[r * kArgmaxChunks + c];
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if (lane == 0) {
    out_idx[r] = bi + index_offset;
    if (out_val) out_val[r] = best;
  }
}

inline int rc() { return (int)cudaGetLastError(); }

}  // namespace

extern "C" {

int b200_rmsnorm(void* x, const void* delta, const float* partials, int splits, const void* gamma,
                 void* out, long long rows, int cols, float eps, int unit_offset, int write_x,
                 cudaStream_t stream) {
  if (cols % 8 || rows <= 0) return -6;
  const int nvec = cols / 8;
  int threads = nvec >= 256 ? 256 : ((nvec + 31) / 32) * 32;
  const int per = (nvec + threads - 1) / threads;
  const size_t stride = (size_t)rows * cols;
  auto X = reinterpret_cast<__nv_bfloat16*>(x);
  auto D = reinterpret_cast<const __nv_bfloat16*>(delta);
  auto G = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto O = reinterpret_cast<__nv_bfloat16*>(out);
#define LAUNCH_RN(MV) rmsnorm_kernel<MV><<<(unsigned)rows, threads, 0, stream>>>(X, D, partials, splits, stride, G, O, cols, eps, unit_offset, write_x)
  if (per <= 1) LAUNCH_RN(1);
  else if (per <= 2) LAUNCH_RN(2);
  else if (per <= 4) LAUNCH_RN(4);
  else if (per <= 8) LAUNCH_RN(8);
  else return -6;
#undef LAUNCH_RN
  return rc();
}

int b200_gated_rmsnorm(const void* x, const void* gate, const void* gamma, void* out, long long nrows,
                       int dim, float eps, int heads, long long gate_ld, cudaStream_t stream) {
  if (dim % 8 || dim > 256) return -6;
  const int wpb = 8;
  gated_rmsnorm_kernel<<<(unsigned)((nrows + wpb - 1) / wpb), wpb * 32, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(gate),
      reinterpret_cast<const __nv_bfloat16*>(gamma), reinterpret_cast<__nv_bfloat16*>(out), (size_t)nrows, dim, eps, heads, (size_t)gate_ld);
  return rc();
}

int b200_embedding(const int* ids, const void* table, void* out, int rows, int hidden, int vocab_lo,
                   int vocab_hi, cudaStream_t stream) {
  if (hidden % 8) return -6;
  embedding_kernel<<<rows, 128, 0, stream>>>(ids, reinterpret_cast<const __nv_bfloat16*>(table),
                                             reinterpret_cast<__nv_bfloat16*>(out), hidden, vocab_lo, vocab_hi);
  return rc();
}

int b200_silu_mul(const void* gate_up, void* out, long long rows, int inter, cudaStream_t stream) {
  if (inter % 8) return -6;
  const size_t nvec = (size_t)rows * (inter / 8);
  const unsigned blocks = (unsigned)((nvec + 255) / 256 > 148 * 16 ? 148 * 16 : (nvec + 255) / 256);
  silu_mul_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(gate_up),
                                              reinterpret_cast<__nv_bfloat16*>(out), (size_t)rows, inter);
  return rc();
}

int b200_sigmoid_mul(const void* x, const void* gate, void* out, long long n, cudaStream_t stream) {
  if (n % 8) return -6;
  const size_t n8 = n / 8;
  const unsigned blocks = (unsigned)((n8 + 255) / 256 > 148 * 16 ? 148 * 16 : (n8 + 255) / 256);
  sigmoid_mul_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                 reinterpret_cast<const __nv_bfloat16*>(gate),
                                                 reinterpret_cast<__nv_bfloat16*>(out), n8);
  return rc();
}

int b200_add(void* y, const void* x, long long n, cudaStream_t stream) {
  if (n % 8) return -6;
  const size_t n8 = n / 8;
  const unsigned blocks = (unsigned)((n8 + 255) / 256 > 148 * 16 ? 148 * 16 : (n8 + 255) / 256);
  add_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<__nv_bfloat16*>(y),
                                         reinterpret_cast<const __nv_bfloat16*>(x), n8);
  return rc();
}

int b200_conv_silu(const void* x, int ldx, const void* w, void* tail, void* y, int ldy, int T, int C,
                   int kw, int update_tail, cudaStream_t stream) {
  if (kw != 4 || C % 8) return -6;
  const int threads = 128;
  const int cblocks = (C / 8 + threads - 1) / threads;
  int t_per_block = T;
  int tblocks = 1;
  if (T > 64) {
    t_per_block = 64;
    tblocks = (T + 63) / 64;
  }
  conv_silu_kernel<4><<<dim3(cblocks, tblocks), threads, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<__nv_bfloat16*>(tail), reinterpret_cast<__nv_bfloat16*>(y), ldy, T, C, t_per_block,
      update_tail);
  if (update_tail && tblocks > 1)
    conv_tail_update_kernel<<<cblocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), ldx,
                                                             reinterpret_cast<__nv_bfloat16*>(tail), T, C, kw);
  return rc();
}

int b200_conv_silu_step(const void* x, int ldx, const void* w, void* tails, long long slot_stride,
                        const int* slot_ids, void* y, int ldy, int B, int C, int kw, cudaStream_t stream) {
  if (kw != 4 || C % 8) return -6;
  const int threads = 128;
  const int cblocks = (C / 8 + threads - 1) / threads;
  conv_silu_step_kernel<4><<<dim3(cblocks, B), threads, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), ldx, reinterpret_cast<const __nv_bfloat16*>(w),
      reinterpret_cast<__nv_bfloat16*>(tails), (size_t)slot_stride, slot_ids,
      reinterpret_cast<__nv_bfloat16*>(y), ldy, C);
  return rc();
}

int b200_gdn_gates(const void* ab, int ld, int a_off, int b_off, const float* a_log, const float* dt_bias,
                   float* g, float* beta, long long rows, int heads, cudaStream_t stream) {
  const size_t n = (size_t)rows * heads;
  gdn_gates_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(ab), ld, a_off, b_off, a_log, dt_bias, g, beta, (size_t)rows, heads);
  return rc();
}

int b200_argmax(const void* logits, int is_f32, int ld, int n, int rows, int index_offset, int* out_idx,
                float* out_val, cudaStream_t stream) {
  if (rows <= kArgmaxMaxRows && n >= 8192) {
    const int chunk = (n + kArgmaxChunks - 1) / kArgmaxChunks;
    const int chunks = (n + chunk - 1) / chunk;
    const dim3 grid(chunks, rows);
    if (is_f32) argmax_chunk_kernel<float><<<grid, 256, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, n, chunk);
    else argmax_chunk_kernel<__nv_bfloat16><<<grid, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, n, chunk);
    argmax_final_kernel<<<rows, 32, 0, stream>>>(chunks, index_offset, out_idx, out_val);
    return rc();
  }
  if (is_f32)
    argmax_kernel<float><<<rows, 1024, 0, stream>>>(reinterpret_cast<const float*>(logits), ld, n, index_offset,
                                                    out_idx, out_val);
  else
    argmax_kernel<__nv_bfloat16><<<rows, 1024, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ld, n,
                                                            index_offset, out_idx, out_val);
  return rc();
}

}  // extern "C"
