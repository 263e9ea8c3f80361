// Attention prologue: per-head RMSNorm of q and k ((1+gamma) or plain gamma),
// partial half-split RoPE over the first `rot` dims, split of the q||gate
// projection layout, and the write of K/V rows into the paged cache.
// One warp per (token, head); lane l owns dims [4l, 4l+4) of a 128-wide head.
//
// Reference behaviour: cpp_engine/backends/cuda/kernels/qwen_half_ops.cu
// (partial_rope :2659-2715, split_q_gate :2716, append_kv paged :2772),
// cuda_ops.cu head_rmsnorm_rope :477-670, src/csrc/minimax_rope_kernel.cu:41-78.
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int D = 128;

struct RopeParams {
  const __nv_bfloat16* q_src; int ldq; int q_off; int q_head_stride;  // head h at q_src[t*ldq + q_off + h*q_head_stride]
  int gate_in_q;                                                        // 1: head block is [q(128) | gate(128)]
  const __nv_bfloat16* k_src; int ldk; int k_off;
  const __nv_bfloat16* v_src; int ldv; int v_off;
  const __nv_bfloat16* q_gamma; const __nv_bfloat16* k_gamma;           // optional [128]
  int unit_offset; float eps;
  const float* inv_freq; int rot; float mscale;
  const int* positions; const int* slots;                               // [T]; slot = block * bs + offset
  __nv_bfloat16* q_out; __nv_bfloat16* gate_out;                        // [T, Hq, 128]
  __nv_bfloat16* k_cache; __nv_bfloat16* v_cache; int bs;               // [nb, Hkv, bs, 128]
  int T, Hq, Hkv;
  // full-width mode (row_ss != null): the RMS statistic of q / k is taken over the whole projection row (all heads,
  // all ranks) and arrives precomputed as sums of squares [T, 2]; gamma is then indexed per head.
  const float* row_ss; float q_full_width, k_full_width; int gamma_head_stride;
};

__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 u = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const float (&f)[4]) {
  __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&a);
  u.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = u;
}

__device__ __forceinline__ void norm_rope(float (&x)[4], const __nv_bfloat16* gamma, int unit_offset, float eps,
                                          const float* inv_freq, int rot, float mscale, int pos, int lane,
                                          float full_ss = -1.f, float full_width = 1.f) {
  if (gamma) {
    float inv;
    if (full_ss >= 0.f) {
      inv = rsqrtf(full_ss / full_width + eps);
    } else {
      float ss = x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      inv = rsqrtf(ss / (float)D + eps);
    }
    float g[4];
    load4(gamma + lane * 4, g);
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = x[i] * inv * (unit_offset ? 1.f + g[i] : g[i]);
  }
  if (rot > 0) {
    const int half = rot >> 1;
    const int partner = half >> 2;  // lanes between a dim and its rotation partner
    float y[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) y[i] = __shfl_xor_sync(0xffffffffu, x[i], partner);
    const int d0 = lane * 4;
    if (d0 < rot) {
      const bool lo = d0 < half;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int fi = (lo ? d0 : d0 - half) + i;
        double a = (double)pos * (double)inv_freq[fi];
        a -= 6.283185307179586 * rint(a * 0.15915494309189535);
        float sn, cs;
        __sincosf((float)a, &sn, &cs);
        sn *= mscale;
        cs *= mscale;
        x[i] = lo ? (x[i] * cs - y[i] * sn) : (x[i] * cs + y[i] * sn);
      }
    }
  }
}

__global__ void qk_norm_rope_append_kernel(RopeParams p) {
  const int lane = threadIdx.x & 31;
  const size_t w = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int heads = p.Hq + 2 * p.Hkv;
  if (w >= (size_t)p.T * heads) return;
  const int t = (int)(w / heads);
  const int hh = (int)(w % heads);
  const int pos = p.positions[t];
  float x[4];
  if (hh < p.Hq) {
    const __nv_bfloat16* src = p.q_src + (size_t)t * p.ldq + p.q_off + (size_t)hh * p.q_head_stride;
    load4(src + lane * 4, x);
    norm_rope(x, p.q_gamma ? p.q_gamma + (size_t)hh * p.gamma_head_stride : nullptr, p.unit_offset, p.eps, p.inv_freq,
              p.rot, p.mscale, pos, lane, p.row_ss ? p.row_ss[2 * t] : -1.f, p.q_full_width);
    store4(p.q_out + ((size_t)t * p.Hq + hh) * D + lane * 4, x);
    if (p.gate_in_q && p.gate_out) {
      const uint2 g = *reinterpret_cast<const uint2*>(src + D + lane * 4);
      *reinterpret_cast<uint2*>(p.gate_out + ((size_t)t * p.Hq + hh) * D + lane * 4) = g;
    }
  } else if (hh < p.Hq + p.Hkv) {
    const int h = hh - p.Hq;
    load4(p.k_src + (size_t)t * p.ldk + p.k_off + h * D + lane * 4, x);
    norm_rope(x, p.k_gamma ? p.k_gamma + (size_t)h * p.gamma_head_stride : nullptr, p.unit_offset, p.eps, p.inv_freq,
              p.rot, p.mscale, pos, lane, p.row_ss ? p.row_ss[2 * t + 1] : -1.f, p.k_full_width);
    const int slot = p.slots[t];
    if (slot >= 0)
      store4(p.k_cache + (((size_t)(slot / p.bs) * p.Hkv + h) * p.bs + slot % p.bs) * D + lane * 4, x);
  } else {
    const int h = hh - p.Hq - p.Hkv;
    const uint2 v = *reinterpret_cast<const uint2*>(p.v_src + (size_t)t * p.ldv + p.v_off + h * D + lane * 4);
    const int slot = p.slots[t];
    if (slot >= 0)
      *reinterpret_cast<uint2*>(p.v_cache + (((size_t)(slot / p.bs) * p.Hkv + h) * p.bs + slot % p.bs) * D + lane * 4) = v;
  }
}

// out[t] = (sum of squares of the q columns, of the k columns) of projection row t; one block per token.
__global__ void qk_sumsq_kernel(const __nv_bfloat16* __restrict__ proj, int ld, int q_off, int q_width, int k_off,
                                int k_width, float* __restrict__ out) {
  const int t = blockIdx.x;
  const __nv_bfloat16* row = proj + (size_t)t * ld;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < q_width; i += blockDim.x) { const float v = __bfloat162float(row[q_off + i]); sq += v * v; }
  for (int i = threadIdx.x; i < k_width; i += blockDim.x) { const float v = __bfloat162float(row[k_off + i]); sk += v * v; }
  __shared__ float red[2][8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) { sq += __shfl_xor_sync(0xffffffffu, sq, o); sk += __shfl_xor_sync(0xffffffffu, sk, o); }
  if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = sq; red[1][threadIdx.x >> 5] = sk; }
  __syncthreads();
  if (threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) { a += red[0][w]; b += red[1][w]; }
    out[2 * t] = a;
    out[2 * t + 1] = b;
  }
}

int launch_rope(RopeParams& p, cudaStream_t stream) {
  const int heads = p.Hq + 2 * p.Hkv;
  const size_t warps = (size_t)p.T * heads;
  const int wpb = 8;
  qk_norm_rope_append_kernel<<<(unsigned)((warps + wpb - 1) / wpb), wpb * 32, 0, stream>>>(p);
  return (int)cudaGetLastError();
}

}  // namespace

// Sums of squares of the q and k parts of each projection row (fp32 [T, 2]); with tensor parallelism the caller adds
// the ranks' partial sums before the normalisation below.
extern "C" int b200_qk_sumsq(const void* proj, int ld, int q_off, int q_width, int k_off, int k_width, float* out, int T,
                             cudaStream_t stream) {
  if (T <= 0 || q_width < 0 || k_width < 0) return -6;
  qk_sumsq_kernel<<<T, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(proj), ld, q_off, q_width, k_off, k_width, out);
  return (int)cudaGetLastError();
}

// Full-width QK RMSNorm variant (MiniMax-style: the statistic spans the whole q / k projection row, gamma has one
// entry per (head, dim)): row_ss holds the rows' sums of squares, q_full_width / k_full_width the element counts they
// were taken over; gamma pointers address this rank's heads, [H, 128].  Otherwise as b200_qk_norm_rope_append.
extern "C" int b200_qk_fullnorm_rope_append(
    const void* q_src, int ldq, int q_off, const void* k_src, int ldk, int k_off, const void* v_src, int ldv, int v_off,
    const void* q_gamma, const void* k_gamma, const float* row_ss, int q_full_width, int k_full_width, float eps,
    const float* inv_freq, int rot, const int* positions, const int* slots, void* q_out, void* k_cache, void* v_cache,
    int block_size, int T, int Hq, int Hkv, cudaStream_t stream) {
  if (rot < 0 || rot > D || (rot & 7) || !row_ss || !q_gamma || !k_gamma) return -6;
  if (rot > 0) {
    const int partner = rot >> 3;
    if (partner & (partner - 1)) return -6;
  }
  RopeParams p;
  p.q_src = reinterpret_cast<const __nv_bfloat16*>(q_src); p.ldq = ldq; p.q_off = q_off; p.q_head_stride = D;
  p.gate_in_q = 0;
  p.k_src = reinterpret_cast<const __nv_bfloat16*>(k_src); p.ldk = ldk; p.k_off = k_off;
  p.v_src = reinterpret_cast<const __nv_bfloat16*>(v_src); p.ldv = ldv; p.v_off = v_off;
  p.q_gamma = reinterpret_cast<const __nv_bfloat16*>(q_gamma);
  p.k_gamma = reinterpret_cast<const __nv_bfloat16*>(k_gamma);
  p.unit_offset = 0; p.eps = eps;
  p.inv_freq = inv_freq; p.rot = rot; p.mscale = 1.f;
  p.positions = positions; p.slots = slots;
  p.q_out = reinterpret_cast<__nv_bfloat16*>(q_out);
  p.gate_out = nullptr;
  p.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache);
  p.bs = block_size; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.row_ss = row_ss; p.q_full_width = (float)q_full_width; p.k_full_width = (float)k_full_width; p.gamma_head_stride = D;
  return launch_rope(p, stream);
}

extern "C" int b200_qk_norm_rope_append(
    const void* q_src, int ldq, int q_off, int q_head_stride, int gate_in_q, const void* k_src, int ldk, int k_off,
    const void* v_src, int ldv, int v_off, const void* q_gamma, const void* k_gamma, int unit_offset, float eps,
    const float* inv_freq, int rot, float mscale, const int* positions, const int* slots, void* q_out,
    void* gate_out, void* k_cache, void* v_cache, int block_size, int T, int Hq, int Hkv, cudaStream_t stream) {
  if (rot < 0 || rot > D || (rot & 7)) return -6;
  if (rot > 0) {
    const int partner = rot >> 3;
    if (partner & (partner - 1)) return -6;  // rotation partner must be a power-of-two lane distance
  }
  RopeParams p;
  p.q_src = reinterpret_cast<const __nv_bfloat16*>(q_src); p.ldq = ldq; p.q_off = q_off; p.q_head_stride = q_head_stride;
  p.gate_in_q = gate_in_q;
  p.k_src = reinterpret_cast<const __nv_bfloat16*>(k_src); p.ldk = ldk; p.k_off = k_off;
  p.v_src = reinterpret_cast<const __nv_bfloat16*>(v_src); p.ldv = ldv; p.v_off = v_off;
  p.q_gamma = reinterpret_cast<const __nv_bfloat16*>(q_gamma);
  p.k_gamma = reinterpret_cast<const __nv_bfloat16*>(k_gamma);
  p.unit_offset = unit_offset; p.eps = eps;
  p.inv_freq = inv_freq; p.rot = rot; p.mscale = mscale;
  p.positions = positions; p.slots = slots;
  p.q_out = reinterpret_cast<__nv_bfloat16*>(q_out);
  p.gate_out = reinterpret_cast<__nv_bfloat16*>(gate_out);
  p.k_cache = reinterpret_cast<__nv_bfloat16*>(k_cache);
  p.v_cache = reinterpret_cast<__nv_bfloat16*>(v_cache);
  p.bs = block_size; p.T = T; p.Hq = Hq; p.Hkv = Hkv;
  p.row_ss = nullptr; p.q_full_width = 1.f; p.k_full_width = 1.f; p.gamma_head_stride = 0;
  return launch_rope(p, stream);
}
