// Fused kernels for the decode step (a handful of tokens per launch), where launch count and
// round trips through HBM dominate the time outside the weight-streaming GEMMs:
//   * gdn_decode_fused   - everything between the qkv|z projection and the output projection of a
//                          Gated DeltaNet layer in one launch: the a/b head projections, the gates
//                          g = -exp(A_log) softplus(a + dt_bias) and beta = sigmoid(b), the causal
//                          depth-wise conv step with its tail update, SiLU, L2-normalised q/k, the
//                          gated delta-rule state update and read-out, and the per-head gated RMSNorm;
//   * rmsnorm_split      - residual add + RMSNorm that also emits the activation as E4M3 terms for
//                          the weight-streaming GEMM (gemm_w8a8s.cu), saving the separate split launch;
//   * silu_mul_split     - SwiGLU activation that emits E4M3 terms directly.
// Reference counterparts are separate kernels per step
// (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu: conv_silu_f16_batched :2233, linear_gates_f16 :2265,
//  gated_delta_step_batched_f16 :2350, gated_rmsnorm_f16 :2163, residual_add_rmsnorm_f16 :2072, silu_mul_f16 :2741).
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "ops.h"
#include "launch.h"

namespace {

constexpr int DK = 128, DV = 128;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

struct GdnDecodeParams {
  const __nv_bfloat16* proj;   // [B, ldp]: q | k | v | z  (q at 0, k at kd, v at 2kd, z at 2kd + vd)
  int ldp;
  const __nv_bfloat16* x;      // [B, hidden] normed layer input (for the a/b projections)
  int hidden;
  const __nv_bfloat16* w_ab;   // [2*Hv, hidden]: rows 0..Hv-1 = a, Hv..2Hv-1 = b
  const float* a_log;          // [Hv]
  const float* dt_bias;        // [Hv]
  const __nv_bfloat16* conv_w; // [C, KW], C = 2kd + vd
  __nv_bfloat16* tails;        // [slots, KW-1, C]
  size_t tail_stride;
  float* states;               // [slots, Hv, 128, 128] at slot_stride
  size_t state_stride;
  const int* slot_ids;         // [B] or null
  const __nv_bfloat16* gamma;  // [128] gated-norm weight
  __nv_bfloat16* out;          // [B, Hv*128]
  int Hv, Hk;
  float eps, q_scale;
};

// One conv step for channel c of row b: y = silu(sum_k w[c][k] * hist[k]); shifts the tail.
template <int KW>
__device__ __forceinline__ float conv_step(const GdnDecodeParams& p, __nv_bfloat16* tail, int C, int c, float cur,
                                           bool write_tail) {
  float h[KW - 1];
#pragma unroll
  for (int k = 0; k < KW - 1; ++k) h[k] = __bfloat162float(tail[(size_t)k * C + c]);
  float acc = cur * __bfloat162float(p.conv_w[(size_t)c * KW + KW - 1]);
#pragma unroll
  for (int k = 0; k < KW - 1; ++k) acc += h[k] * __bfloat162float(p.conv_w[(size_t)c * KW + k]);
  if (write_tail) {
#pragma unroll
    for (int k = 0; k + 1 < KW - 1; ++k) tail[(size_t)k * C + c] = __float2bfloat16(h[k + 1]);
    tail[(size_t)(KW - 2) * C + c] = __float2bfloat16(cur);
  }
  // the unfused path stores the conv output as bf16 before the recurrence reads it
  return bf16_round(silu_f(acc));
}

// grid (Hk, B); block = 128 * R * RG threads (R = Hv / Hk value heads per key head, RG row groups).
// Thread (grp, rg, j) owns rows [rg*128/RG, (rg+1)*128/RG) of state column j of value head kh*R + grp; the row
// groups cut the serial length of the recurrence per thread, their partial dot products meet in shared memory.
// The q/k channels of key head kh are convolved once, by the threads with grp == 0 and rg == 0.
template <int KW, int R, int RG>
__global__ void __launch_bounds__(128 * R * RG)
gdn_decode_fused_kernel(GdnDecodeParams p) {
  constexpr int ROWS = DK / RG;
  constexpr int WPH = 4 * RG;              // warps per value head
  __shared__ float sq[DK], sk[DK];
  __shared__ float s_v[R][DV];
  __shared__ float s_part[R][RG][DV];
  __shared__ float red_ab[R][WPH][2];
  __shared__ float red_qk[8];
  __shared__ float red_o[R][4];
  __shared__ float s_gate[R][2];
  b200::pdl_grid_trigger();
  b200::pdl_grid_wait();
  const int kh = blockIdx.x, b = blockIdx.y;
  const int j = threadIdx.x & 127;
  const int rg = (threadIdx.x >> 7) % RG;
  const int grp = threadIdx.x / (128 * RG);
  const int h = kh * R + grp;
  const int kd = p.Hk * DK, vd = p.Hv * DV, C = 2 * kd + vd;
  const int slot = p.slot_ids ? p.slot_ids[b] : b;
  __nv_bfloat16* tail = p.tails + (size_t)slot * p.tail_stride;
  const __nv_bfloat16* row = p.proj + (size_t)b * p.ldp;

  // ---- a/b projections of this value head: two dot products of length hidden over the head's 128*RG threads
  {
    const __nv_bfloat16* xr = p.x + (size_t)b * p.hidden;
    const __nv_bfloat16* wa = p.w_ab + (size_t)h * p.hidden;
    const __nv_bfloat16* wb = p.w_ab + (size_t)(p.Hv + h) * p.hidden;
    float da = 0.f, db = 0.f;
    for (int i = (rg * 128 + j) * 8; i < p.hidden; i += 128 * RG * 8) {
      const uint4 xv = *reinterpret_cast<const uint4*>(xr + i);
      const uint4 av = *reinterpret_cast<const uint4*>(wa + i);
      const uint4 bv = *reinterpret_cast<const uint4*>(wb + i);
      const __nv_bfloat162* xh = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
      const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 xf = __bfloat1622float2(xh[e]), af = __bfloat1622float2(ah[e]), bf = __bfloat1622float2(bh[e]);
        da += xf.x * af.x + xf.y * af.y;
        db += xf.x * bf.x + xf.y * bf.y;
      }
    }
    da = warp_sum(da);
    db = warp_sum(db);
    if ((j & 31) == 0) {
      red_ab[grp][rg * 4 + (j >> 5)][0] = da;
      red_ab[grp][rg * 4 + (j >> 5)][1] = db;
    }
  }
  // ---- conv step (row group 0 only): q/k channels by value head 0 of the block, v channel by every head
  float qv = 0.f, kv = 0.f;
  if (rg == 0) {
    if (grp == 0) {
      qv = conv_step<KW>(p, tail, C, kh * DK + j, __bfloat162float(row[kh * DK + j]), true);
      kv = conv_step<KW>(p, tail, C, kd + kh * DK + j, __bfloat162float(row[kd + kh * DK + j]), true);
      const float qs = warp_sum(qv * qv), ks = warp_sum(kv * kv);
      if ((j & 31) == 0) {
        red_qk[j >> 5] = qs;
        red_qk[4 + (j >> 5)] = ks;
      }
    }
    s_v[grp][j] = conv_step<KW>(p, tail, C, 2 * kd + h * DV + j, __bfloat162float(row[2 * kd + h * DV + j]), true);
  }
  __syncthreads();
  if (rg == 0 && j == 0) {
    float a = 0.f, bb = 0.f;
#pragma unroll
    for (int w = 0; w < WPH; ++w) {
      a += red_ab[grp][w][0];
      bb += red_ab[grp][w][1];
    }
    // the unfused path rounds the a/b projection outputs to bf16 before the gate math
    a = bf16_round(a);
    bb = bf16_round(bb);
    const float av = a + p.dt_bias[h];
    const float sp = av > 20.f ? av : log1pf(expf(av));
    s_gate[grp][0] = __expf(-expf(p.a_log[h]) * sp);   // decay = exp(g)
    s_gate[grp][1] = sigmoid_f(bb);
  }
  if (grp == 0 && rg == 0) {
    const float qn = rsqrtf(red_qk[0] + red_qk[1] + red_qk[2] + red_qk[3] + 1e-6f);
    const float kn = rsqrtf(red_qk[4] + red_qk[5] + red_qk[6] + red_qk[7] + 1e-6f);
    sq[j] = qv * qn * p.q_scale;
    sk[j] = kv * kn;
  }
  __syncthreads();
  // ---- gated delta rule on rows [rg*ROWS, (rg+1)*ROWS) of state column j of head h
  float* S = p.states + (size_t)slot * p.state_stride + (size_t)h * DK * DV + (size_t)rg * ROWS * DV;
  const float decay = s_gate[grp][0], bt = s_gate[grp][1];
  float col[ROWS];
  float part = 0.f;
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    col[i] = S[(size_t)i * DV + j] * decay;
    part += col[i] * sk[rg * ROWS + i];
  }
  s_part[grp][rg][j] = part;
  __syncthreads();
  float kv_mem = 0.f;
#pragma unroll
  for (int g2 = 0; g2 < RG; ++g2) kv_mem += s_part[grp][g2][j];
  const float delta = (s_v[grp][j] - kv_mem) * bt;
  __syncthreads();   // s_part is reused for the read-out partials
  part = 0.f;
#pragma unroll
  for (int i = 0; i < ROWS; ++i) {
    col[i] += sk[rg * ROWS + i] * delta;
    S[(size_t)i * DV + j] = col[i];
    part += col[i] * sq[rg * ROWS + i];
  }
  s_part[grp][rg][j] = part;
  __syncthreads();
  // ---- per-head gated RMSNorm by row group 0 (the unfused path stores o as bf16 first)
  float o = 0.f;
  if (rg == 0) {
#pragma unroll
    for (int g2 = 0; g2 < RG; ++g2) o += s_part[grp][g2][j];
    o = bf16_round(o);
    const float ss = warp_sum(o * o);
    if ((j & 31) == 0) red_o[grp][j >> 5] = ss;
  }
  __syncthreads();
  if (rg == 0) {
    const float inv = rsqrtf((red_o[grp][0] + red_o[grp][1] + red_o[grp][2] + red_o[grp][3]) / (float)DV + p.eps);
    const float z = __bfloat162float(row[2 * kd + vd + h * DV + j]);
    const float y = o * inv * __bfloat162float(p.gamma[j]) * silu_f(z);
    p.out[((size_t)b * p.Hv + h) * DV + j] = __float2bfloat16(y);
  }
}

// ------------------------------------------------------------------------------------------------
// E4M3 term split of one value already scaled by the row scale; byte order (x0,x2,x1,x3) per 4 values.
template <int TERMS>
__device__ __forceinline__ void split4_store(float (&v)[4], uint8_t* xq_row0, size_t term_stride, int i) {
#pragma unroll
  for (int t = 0; t < TERMS; ++t) {
    uint8_t q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __nv_fp8_e4m3 f8(v[e]);
      q[e] = f8.__x;
      v[e] = (v[e] - float(f8)) * 16.f;
    }
    *reinterpret_cast<uint32_t*>(xq_row0 + t * term_stride + i) =
        (uint32_t)q[0] | ((uint32_t)q[2] << 8) | ((uint32_t)q[1] << 16) | ((uint32_t)q[3] << 24);
  }
}

__device__ __forceinline__ float block_max(float v, float* red) {
  v = warp_max(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_max(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  __syncthreads();
  return t;
}
__device__ __forceinline__ float block_sum2(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  __syncthreads();
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

// One block per row, 4 values per thread per step; cols % 4 == 0, cols <= 4 * MAXV * blockDim.
template <int MAXV, int TERMS>
__global__ void rmsnorm_split_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ delta,
                                     const __nv_bfloat16* __restrict__ gamma, __nv_bfloat16* __restrict__ out,
                                     uint8_t* __restrict__ xq, float* __restrict__ inv_c, int cols, float eps,
                                     int unit_offset) {
  __shared__ float red[32];
  b200::pdl_grid_trigger();   // the GEMM that follows may start streaming its weights now
  b200::pdl_grid_wait();
  const size_t row = blockIdx.x;
  float cache[MAXV][4];
  float ss = 0.f;
#pragma unroll
  for (int it = 0; it < MAXV; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    if (i < cols) {
      const uint2 u = *reinterpret_cast<const uint2*>(x + row * cols + i);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
      float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
      if (delta) {
        const uint2 d = *reinterpret_cast<const uint2*>(delta + row * cols + i);
        const __nv_bfloat162* dh = reinterpret_cast<const __nv_bfloat162*>(&d);
        const float2 da = __bfloat1622float2(dh[0]), db = __bfloat1622float2(dh[1]);
        // the residual stream is bf16: round first so the norm input equals the stored residual
        uint2 r;
        __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&r);
        rh[0] = __floats2bfloat162_rn(a.x + da.x, a.y + da.y);
        rh[1] = __floats2bfloat162_rn(b.x + db.x, b.y + db.y);
        *reinterpret_cast<uint2*>(x + row * cols + i) = r;
        a = __bfloat1622float2(rh[0]);
        b = __bfloat1622float2(rh[1]);
      }
      cache[it][0] = a.x; cache[it][1] = a.y; cache[it][2] = b.x; cache[it][3] = b.y;
      ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
    }
  }
  const float inv = rsqrtf(block_sum2(ss, red) / (float)cols + eps);
  float m = 0.f;
#pragma unroll
  for (int it = 0; it < MAXV; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    if (i < cols) {
      const uint2 g = *reinterpret_cast<const uint2*>(gamma + i);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
      const float2 g0 = __bfloat1622float2(gh[0]), g1 = __bfloat1622float2(gh[1]);
      const float gf[4] = {g0.x, g0.y, g1.x, g1.y};
      uint2 r;
      __nv_bfloat162* rh = reinterpret_cast<__nv_bfloat162*>(&r);
      float o[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) o[e] = cache[it][e] * inv * (unit_offset ? 1.f + gf[e] : gf[e]);
      rh[0] = __floats2bfloat162_rn(o[0], o[1]);
      rh[1] = __floats2bfloat162_rn(o[2], o[3]);
      if (out) *reinterpret_cast<uint2*>(out + row * cols + i) = r;
      const float2 q0 = __bfloat1622float2(rh[0]), q1 = __bfloat1622float2(rh[1]);
      cache[it][0] = q0.x; cache[it][1] = q0.y; cache[it][2] = q1.x; cache[it][3] = q1.y;
      m = fmaxf(m, fmaxf(fmaxf(fabsf(q0.x), fabsf(q0.y)), fmaxf(fabsf(q1.x), fabsf(q1.y))));
    }
  }
  m = block_max(m, red);
  const float c = m > 0.f ? 224.f / m : 1.f;
  if (threadIdx.x == 0) inv_c[row] = 1.f / c;
#pragma unroll
  for (int it = 0; it < MAXV; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    if (i < cols) {
      float v[4] = {cache[it][0] * c, cache[it][1] * c, cache[it][2] * c, cache[it][3] * c};
      split4_store<TERMS>(v, xq + row * TERMS * (size_t)cols, (size_t)cols, i);
    }
  }
}

// act[t, i] = silu(gu[t, i]) * gu[t, inter + i]; one block per row; inter % 4 == 0, inter <= 4 * MAXV * blockDim.
template <int MAXV, int TERMS>
__global__ void silu_mul_split_kernel(const __nv_bfloat16* __restrict__ gu, int inter, uint8_t* __restrict__ xq,
                                      float* __restrict__ inv_c) {
  __shared__ float red[32];
  b200::pdl_grid_trigger();   // the GEMM that follows may start streaming its weights now
  b200::pdl_grid_wait();
  const size_t row = blockIdx.x;
  const __nv_bfloat16* g = gu + row * 2 * (size_t)inter;
  const __nv_bfloat16* u = g + inter;
  float cache[MAXV][4];
  float m = 0.f;
#pragma unroll
  for (int it = 0; it < MAXV; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    if (i < inter) {
      const uint2 gv = *reinterpret_cast<const uint2*>(g + i);
      const uint2 uv = *reinterpret_cast<const uint2*>(u + i);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
      const __nv_bfloat162* uh = reinterpret_cast<const __nv_bfloat162*>(&uv);
      const float2 g0 = __bfloat1622float2(gh[0]), g1 = __bfloat1622float2(gh[1]);
      const float2 u0 = __bfloat1622float2(uh[0]), u1 = __bfloat1622float2(uh[1]);
      cache[it][0] = bf16_round(silu_f(g0.x) * u0.x);
      cache[it][1] = bf16_round(silu_f(g0.y) * u0.y);
      cache[it][2] = bf16_round(silu_f(g1.x) * u1.x);
      cache[it][3] = bf16_round(silu_f(g1.y) * u1.y);
#pragma unroll
      for (int e = 0; e < 4; ++e) m = fmaxf(m, fabsf(cache[it][e]));
    }
  }
  m = block_max(m, red);
  const float c = m > 0.f ? 224.f / m : 1.f;
  if (threadIdx.x == 0) inv_c[row] = 1.f / c;
#pragma unroll
  for (int it = 0; it < MAXV; ++it) {
    const int i = (threadIdx.x + it * blockDim.x) * 4;
    if (i < inter) {
      float v[4] = {cache[it][0] * c, cache[it][1] * c, cache[it][2] * c, cache[it][3] * c};
      split4_store<TERMS>(v, xq + row * TERMS * (size_t)inter, (size_t)inter, i);
    }
  }
}

}  // namespace

extern "C" {

// proj: [B, ldp] bf16 holding q | k | v | z at offsets 0, kd, 2kd, 2kd+vd (kd = Hk*128, vd = Hv*128);
// x: [B, hidden] bf16; w_ab: [2*Hv, hidden] bf16; conv_w: [2kd+vd, kw] bf16; tails: [slots, kw-1, 2kd+vd] bf16
// (tail_stride elements per slot); states: fp32 [slots, Hv, 128, 128] (state_stride floats per slot);
// out: [B, Hv*128] bf16.  Hv / Hk must be 1, 2 or 4 and kw == 4.
int b200_gdn_decode_fused(const void* proj, int ldp, const void* x, int hidden, const void* w_ab, const float* a_log,
                          const float* dt_bias, const void* conv_w, int kw, void* tails, long long tail_stride,
                          float* states, long long state_stride, const int* slot_ids, const void* gamma, void* out,
                          int B, int Hv, int Hk, float eps, cudaStream_t stream) {
  if (B <= 0 || Hv <= 0 || Hk <= 0 || Hv % Hk != 0 || kw != 4 || hidden % 8 != 0) return -6;
  GdnDecodeParams p;
  p.proj = reinterpret_cast<const __nv_bfloat16*>(proj);
  p.ldp = ldp;
  p.x = reinterpret_cast<const __nv_bfloat16*>(x);
  p.hidden = hidden;
  p.w_ab = reinterpret_cast<const __nv_bfloat16*>(w_ab);
  p.a_log = a_log;
  p.dt_bias = dt_bias;
  p.conv_w = reinterpret_cast<const __nv_bfloat16*>(conv_w);
  p.tails = reinterpret_cast<__nv_bfloat16*>(tails);
  p.tail_stride = (size_t)tail_stride;
  p.states = states;
  p.state_stride = (size_t)state_stride;
  p.slot_ids = slot_ids;
  p.gamma = reinterpret_cast<const __nv_bfloat16*>(gamma);
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.Hv = Hv;
  p.Hk = Hk;
  p.eps = eps;
  p.q_scale = rsqrtf((float)DK);
  const dim3 grid(Hk, B);
  switch (Hv / Hk) {
    case 1: return (int)b200::launch_pdl(gdn_decode_fused_kernel<4, 1, 4>, grid, dim3(512), 0, stream, p);
    case 2: return (int)b200::launch_pdl(gdn_decode_fused_kernel<4, 2, 4>, grid, dim3(1024), 0, stream, p);
    case 4: return (int)b200::launch_pdl(gdn_decode_fused_kernel<4, 4, 2>, grid, dim3(1024), 0, stream, p);
    default: return -6;
  }
}

// x[T, cols] (+= delta, written back when delta is given) -> out = rmsnorm(x) * gamma (bf16, optional) and the
// E4M3 terms of that bf16 result: xq [T*terms, cols], inv_c [T].  cols % 4 == 0, cols <= 16384.
int b200_rmsnorm_split(void* x, const void* delta, const void* gamma, void* out, void* xq, float* inv_c, int T,
                       int cols, float eps, int unit_offset, int terms, cudaStream_t stream) {
  if (T <= 0 || cols <= 0 || cols % 4 != 0 || cols > 16384 || (terms != 2 && terms != 3)) return -6;
  auto* xp = reinterpret_cast<__nv_bfloat16*>(x);
  auto* dp = reinterpret_cast<const __nv_bfloat16*>(delta);
  auto* gp = reinterpret_cast<const __nv_bfloat16*>(gamma);
  auto* op = reinterpret_cast<__nv_bfloat16*>(out);
  auto* qp = reinterpret_cast<uint8_t*>(xq);
  const int threads = cols <= 4096 ? 256 : 512;
  if (terms == 3)
    return (int)b200::launch_pdl(rmsnorm_split_kernel<8, 3>, dim3(T), dim3(threads), 0, stream, xp, dp, gp, op, qp, inv_c,
                                 cols, eps, unit_offset);
  return (int)b200::launch_pdl(rmsnorm_split_kernel<8, 2>, dim3(T), dim3(threads), 0, stream, xp, dp, gp, op, qp, inv_c,
                               cols, eps, unit_offset);
}

// gu[T, 2*inter] (gate | up) -> E4M3 terms of bf16(silu(gate) * up): xq [T*terms, inter], inv_c [T].
int b200_silu_mul_split(const void* gu, void* xq, float* inv_c, int T, int inter, int terms, cudaStream_t stream) {
  if (T <= 0 || inter <= 0 || inter % 4 != 0 || inter > 4 * 8 * 1024 || (terms != 2 && terms != 3)) return -6;
  auto* gp = reinterpret_cast<const __nv_bfloat16*>(gu);
  auto* qp = reinterpret_cast<uint8_t*>(xq);
  if (terms == 3) return (int)b200::launch_pdl(silu_mul_split_kernel<8, 3>, dim3(T), dim3(1024), 0, stream, gp, inter, qp, inv_c);
  return (int)b200::launch_pdl(silu_mul_split_kernel<8, 2>, dim3(T), dim3(1024), 0, stream, gp, inter, qp, inv_c);
}

}  // extern "C"
