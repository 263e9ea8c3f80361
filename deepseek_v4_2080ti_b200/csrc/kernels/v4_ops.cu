// Small fused kernels of the DeepSeek-V4 block structure:
//   hadamard128   - orthonormal Walsh-Hadamard rotation of 128-wide bf16 rows (one warp per row, butterflies through
//                   registers and shuffles);
//   hc_split_pre  - hyper-connection input mixer for 4 streams: per token, the 24 mixing logits become pre / post
//                   weights and a 4x4 combination matrix made doubly stochastic by Sinkhorn iterations, and the
//                   sub-layer input y = sum_j pre[j] x[j] is formed in the same pass over the streams;
//   hc_post       - write-back: out[i] = post[i] y + sum_j comb[j][i] residual[j].
// Reference behaviour: hadamard128_forward, hc_split_pre_forward, hc_post_forward of the torch extension
// (src/csrc/cuda_kernel.cpp:2197-2254 op list; math in src/kernels/ops.py:1224-1250 and
// src/models/deepseek_v4/runtime.py:4369-4437).
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops.h"

namespace {

__global__ void hadamard128_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long long rows) {
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint2 u = *reinterpret_cast<const uint2*>(x + row * 128 + lane * 4);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
  float v[4] = {a.x, a.y, b.x, b.y};
  // strides 1 and 2 inside the lane
  float t0 = v[0] + v[1], t1 = v[0] - v[1], t2 = v[2] + v[3], t3 = v[2] - v[3];
  v[0] = t0 + t2; v[1] = t1 + t3; v[2] = t0 - t2; v[3] = t1 - t3;
  // strides 4 .. 64 across lanes
#pragma unroll
  for (int m = 1; m < 32; m <<= 1) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float o = __shfl_xor_sync(0xffffffffu, v[i], m);
      v[i] = (lane & m) ? o - v[i] : v[i] + o;
    }
  }
  const float s = 0.08838834764831845f;   // 128^-1/2
  __nv_bfloat162 r0 = __floats2bfloat162_rn(v[0] * s, v[1] * s), r1 = __floats2bfloat162_rn(v[2] * s, v[3] * s);
  uint2 o;
  o.x = *reinterpret_cast<uint32_t*>(&r0);
  o.y = *reinterpret_cast<uint32_t*>(&r1);
  *reinterpret_cast<uint2*>(y + row * 128 + lane * 4) = o;
}

// mixes fp32 [T, 24]; x bf16 [T, 4, D]; scale fp32 [3]; base fp32 [24].  y bf16 [T, D]; post fp32 [T, 4]; comb fp32 [T, 16].
__global__ void __launch_bounds__(256)
hc_split_pre_kernel(const float* __restrict__ mixes, const __nv_bfloat16* __restrict__ x, const float* __restrict__ scale,
                    const float* __restrict__ base, int D, int iters, float eps, __nv_bfloat16* __restrict__ y,
                    float* __restrict__ post, float* __restrict__ comb) {
  __shared__ float pre_s[4];
  const long long t = blockIdx.x;
  if (threadIdx.x == 0) {
    const float* m = mixes + t * 24;
    for (int i = 0; i < 4; ++i) {
      pre_s[i] = 1.f / (1.f + __expf(-(m[i] * scale[0] + base[i]))) + eps;
      post[t * 4 + i] = 2.f / (1.f + __expf(-(m[4 + i] * scale[1] + base[4 + i])));
    }
    float c[4][4];
    for (int i = 0; i < 4; ++i) {
      float mx = -INFINITY, sum = 0.f;
      for (int j = 0; j < 4; ++j) { c[i][j] = m[8 + 4 * i + j] * scale[2] + base[8 + 4 * i + j]; mx = fmaxf(mx, c[i][j]); }
      for (int j = 0; j < 4; ++j) { c[i][j] = __expf(c[i][j] - mx); sum += c[i][j]; }
      for (int j = 0; j < 4; ++j) c[i][j] = c[i][j] / sum + eps;
    }
    for (int j = 0; j < 4; ++j) {                           // columns
      const float s = c[0][j] + c[1][j] + c[2][j] + c[3][j] + eps;
      for (int i = 0; i < 4; ++i) c[i][j] /= s;
    }
    for (int it = 1; it < iters; ++it) {
      for (int i = 0; i < 4; ++i) {
        const float s = c[i][0] + c[i][1] + c[i][2] + c[i][3] + eps;
        for (int j = 0; j < 4; ++j) c[i][j] /= s;
      }
      for (int j = 0; j < 4; ++j) {
        const float s = c[0][j] + c[1][j] + c[2][j] + c[3][j] + eps;
        for (int i = 0; i < 4; ++i) c[i][j] /= s;
      }
    }
    for (int i = 0; i < 4; ++i)
      for (int j = 0; j < 4; ++j) comb[t * 16 + 4 * i + j] = c[i][j];
  }
  __syncthreads();
  const __nv_bfloat16* xt = x + t * 4 * (long long)D;
  for (int d = threadIdx.x * 2; d < D; d += blockDim.x * 2) {
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(xt + (long long)j * D + d));
      a0 += pre_s[j] * f.x;
      a1 += pre_s[j] * f.y;
    }
    *reinterpret_cast<__nv_bfloat162*>(y + t * D + d) = __floats2bfloat162_rn(a0, a1);
  }
}

// y bf16 [T, D]; residual bf16 [T, 4, D]; post fp32 [T, 4]; comb fp32 [T, 16] (comb[j][i]).  out bf16 [T, 4, D].
__global__ void __launch_bounds__(256)
hc_post_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ residual, const float* __restrict__ post,
               const float* __restrict__ comb, int D, __nv_bfloat16* __restrict__ out) {
  __shared__ float p[4], c[16];
  const long long t = blockIdx.x;
  if (threadIdx.x < 4) p[threadIdx.x] = post[t * 4 + threadIdx.x];
  if (threadIdx.x < 16) c[threadIdx.x] = comb[t * 16 + threadIdx.x];
  __syncthreads();
  for (int d = threadIdx.x * 2; d < D; d += blockDim.x * 2) {
    const float2 yv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(y + t * D + d));
    float2 r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      r[j] = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(residual + (t * 4 + j) * (long long)D + d));
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a0 = p[i] * yv.x, a1 = p[i] * yv.y;
#pragma unroll
      for (int j = 0; j < 4; ++j) { a0 += c[4 * j + i] * r[j].x; a1 += c[4 * j + i] * r[j].y; }
      *reinterpret_cast<__nv_bfloat162*>(out + (t * 4 + i) * (long long)D + d) = __floats2bfloat162_rn(a0, a1);
    }
  }
}

}  // namespace

extern "C" {

int b200_hadamard128(const void* x, void* y, long long rows, cudaStream_t stream) {
  if (rows <= 0) return -6;
  hadamard128_kernel<<<(unsigned)((rows + 7) / 8), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x),
                                                                     reinterpret_cast<__nv_bfloat16*>(y), rows);
  return (int)cudaGetLastError();
}

int b200_hc_split_pre(const float* mixes, const void* x, const float* scale, const float* base, long long T, int D, int iters,
                      float eps, void* y, float* post, float* comb, cudaStream_t stream) {
  if (T <= 0 || D <= 0 || (D & 1)) return -6;
  hc_split_pre_kernel<<<(unsigned)T, 256, 0, stream>>>(mixes, reinterpret_cast<const __nv_bfloat16*>(x), scale, base, D, iters,
                                                        eps, reinterpret_cast<__nv_bfloat16*>(y), post, comb);
  return (int)cudaGetLastError();
}

int b200_hc_post(const void* y, const void* residual, const float* post, const float* comb, long long T, int D, void* out,
                 cudaStream_t stream) {
  if (T <= 0 || D <= 0 || (D & 1)) return -6;
  hc_post_kernel<<<(unsigned)T, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(y),
                                                   reinterpret_cast<const __nv_bfloat16*>(residual), post, comb, D,
                                                   reinterpret_cast<__nv_bfloat16*>(out));
  return (int)cudaGetLastError();
}

}  // extern "C"
