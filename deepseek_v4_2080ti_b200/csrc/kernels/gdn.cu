// Gated DeltaNet (gated delta rule) for head dims dk = dv = 128:
//   * gdn_step    - single-token recurrence for decode batches (one state per slot);
//   * gdn_prepare - chunk-parallel part of the chunked scan (chunk 64): L2-normalised
//                   q/k, in-chunk cumulative log-decay, the (I - A)^-1 "UT transform"
//                   by forward substitution, U = T (beta v), W = T (beta e^gc k),
//                   and the decayed q k^T block;
//   * gdn_scan    - the sequential inter-chunk recurrence, one CTA per (head, 32-wide
//                   value slice): v_new = U - W S, O = (q e^gc) S + Aqk v_new,
//                   S = S e^gc_last + (k e^(gc_last-gc))^T v_new.  The four products of a
//                   chunk run on the tensor cores (m16n8k16, fp16 operands, fp32
//                   accumulation); the state lives in fp32 accumulator registers for the
//                   whole call and only an fp16 operand copy is refreshed per chunk; the
//                   next chunk's operands are prefetched with cp.async while the current
//                   one is multiplied.  The chain is latency-bound (128 dependent steps
//                   for 8192 tokens), so the step time, not the FLOP rate, is what counts.
// The chunked form is algebraically the recurrence
//   S_t = e^{g_t} S_{t-1} + k_t (beta_t (v_t - (e^{g_t} S_{t-1})^T k_t))^T,  o_t = S_t^T q_t / sqrt(dk)
// and replaces the reference's per-token serial kernels
// (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:2282-2600, qwen_gdn_flashqla.cu:36);
// the math oracle is the chunked PyTorch form src/models/qwen4_exp/attention.py:184-270.
#include <cuda_bf16.h>
#include "per_device.h"
#include <cuda_fp16.h>
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int DK = 128, DV = 128, C = 64;
constexpr int KP = 132;   // padded row length (floats) for k/q tiles in shared memory
constexpr int AP = 65;    // padded row length for the 64x64 triangular matrices

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ decode step
// grid (Hv, B), 128 threads: thread j owns state column j (all dk rows) in registers.
__global__ void __launch_bounds__(128)
gdn_step_kernel(float* __restrict__ states, size_t slot_stride, const int* __restrict__ slot_ids,
                const __nv_bfloat16* __restrict__ mixed, int ld, int q_off, int k_off, int v_off,
                const float* __restrict__ g, const float* __restrict__ beta, __nv_bfloat16* __restrict__ out,
                int Hv, int Hk, float q_scale) {
  __shared__ float sq[DK], sk[DK];
  const int h = blockIdx.x, b = blockIdx.y, j = threadIdx.x;
  const int kh = h / (Hv / Hk);
  const __nv_bfloat16* row = mixed + (size_t)b * ld;
  const float qv = __bfloat162float(row[q_off + kh * DK + j]);
  const float kv = __bfloat162float(row[k_off + kh * DK + j]);
  __shared__ float red[8];
  float qs = warp_sum(qv * qv), ks = warp_sum(kv * kv);
  if ((j & 31) == 0) { red[j >> 5] = qs; red[4 + (j >> 5)] = ks; }
  __syncthreads();
  const float qn = rsqrtf(red[0] + red[1] + red[2] + red[3] + 1e-6f);
  const float kn = rsqrtf(red[4] + red[5] + red[6] + red[7] + 1e-6f);
  sq[j] = qv * qn * q_scale;
  sk[j] = kv * kn;
  __syncthreads();
  float* S = states + (size_t)(slot_ids ? slot_ids[b] : b) * slot_stride + (size_t)h * DK * DV;
  const float decay = __expf(g[(size_t)b * Hv + h]);
  const float bt = beta[(size_t)b * Hv + h];
  float col[DK];
  float kv_mem = 0.f;
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    col[i] = S[(size_t)i * DV + j] * decay;
    kv_mem += col[i] * sk[i];
  }
  const float delta = (__bfloat162float(row[v_off + h * DV + j]) - kv_mem) * bt;
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < DK; ++i) {
    col[i] += sk[i] * delta;
    S[(size_t)i * DV + j] = col[i];
    o += col[i] * sq[i];
  }
  out[((size_t)b * Hv + h) * DV + j] = __float2bfloat16(o);
}

// ------------------------------------------------------------- chunk preparation
// Workspace rows are indexed by padded token (nchunks * 64) and value head.
// The tensor-core operands are stored as fp16: every one of them is a product of L2-normalised vectors, decays in
// (0, 1] and beta in (0, 1), so fp16's range is ample and its 11-bit significand matches tf32.
struct PrepOut {
  float* U;     // [Tp, Hv, 128]            T (beta v)
  __half* W;    // [Tp, Hv, 128]            T (beta e^gc k)
  __half* Qg;   // [Tp, Hv, 128]            q_hat * scale * e^gc
  __half* KgT;  // [nchunks, Hv, 128, 64]   (k_hat * e^(gc_last - gc))^T: key dim major, token minor
  __half* Aqk;  // [Tp, Hv, 64]             (q_hat*scale . k_hat) e^(gc_i - gc_j), j <= i
  float* Gl;    // [nchunks, Hv]            e^gc_last
};

__global__ void __launch_bounds__(256, 2)
gdn_prepare_kernel(const __nv_bfloat16* __restrict__ mixed, int ld, int q_off, int k_off, int v_off,
                   const float* __restrict__ g, const float* __restrict__ beta, PrepOut o, int T, int Hv, int Hk,
                   float q_scale) {
  extern __shared__ float sm[];
  float* sk = sm;                    // [64][KP]
  float* sq = sk + C * KP;           // [64][KP]
  float* sA = sq + C * KP;           // [64][AP]
  float* sgc = sA + C * AP;          // [64] cumulative log decay
  float* sbeta = sgc + C;            // [64]
  __nv_bfloat16* sv = reinterpret_cast<__nv_bfloat16*>(sbeta + C);  // [64][128]
  const int h = blockIdx.x, c = blockIdx.y;
  const int kh = h / (Hv / Hk);
  const int t0 = c * C;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // load + normalise rows: warp w handles rows w, w+8, ...
  for (int r = warp; r < C; r += 8) {
    const int t = t0 + r;
    float kf[4] = {0, 0, 0, 0}, qf[4] = {0, 0, 0, 0};
    uint2 vraw = make_uint2(0, 0);
    if (t < T) {
      const __nv_bfloat16* row = mixed + (size_t)t * ld;
      const uint2 ku = *reinterpret_cast<const uint2*>(row + k_off + kh * DK + lane * 4);
      const uint2 qu = *reinterpret_cast<const uint2*>(row + q_off + kh * DK + lane * 4);
      vraw = *reinterpret_cast<const uint2*>(row + v_off + h * DV + lane * 4);
      const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&ku);
      const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qu);
      float2 a = __bfloat1622float2(k2[0]), bb = __bfloat1622float2(k2[1]);
      kf[0] = a.x; kf[1] = a.y; kf[2] = bb.x; kf[3] = bb.y;
      a = __bfloat1622float2(q2[0]); bb = __bfloat1622float2(q2[1]);
      qf[0] = a.x; qf[1] = a.y; qf[2] = bb.x; qf[3] = bb.y;
    }
    const float kn = rsqrtf(warp_sum(kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3]) + 1e-6f);
    const float qn = rsqrtf(warp_sum(qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3]) + 1e-6f) * q_scale;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      sk[r * KP + lane * 4 + i] = kf[i] * kn;
      sq[r * KP + lane * 4 + i] = qf[i] * qn;
    }
    *reinterpret_cast<uint2*>(sv + r * DV + lane * 4) = vraw;
  }
  if (warp == 0) {
    // inclusive scan of g over the 64 rows (2 per lane)
    const int ta = t0 + lane, tb = t0 + 32 + lane;
    float ga = ta < T ? g[(size_t)ta * Hv + h] : 0.f;
    float gb = tb < T ? g[(size_t)tb * Hv + h] : 0.f;
#pragma unroll
    for (int ofs = 1; ofs < 32; ofs <<= 1) {
      const float x = __shfl_up_sync(0xffffffffu, ga, ofs);
      const float y = __shfl_up_sync(0xffffffffu, gb, ofs);
      if (lane >= ofs) { ga += x; gb += y; }
    }
    gb += __shfl_sync(0xffffffffu, ga, 31);
    sgc[lane] = ga;
    sgc[32 + lane] = gb;
    sbeta[lane] = ta < T ? beta[(size_t)ta * Hv + h] : 0.f;
    sbeta[32 + lane] = tb < T ? beta[(size_t)tb * Hv + h] : 0.f;
  }
  __syncthreads();

  // k k^T and q k^T blocks: thread -> 4x4 tile
  {
    const int ti = tid >> 4, tj = tid & 15;
    float akk[4][4], aqk[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b2 = 0; b2 < 4; ++b2) akk[a][b2] = aqk[a][b2] = 0.f;
    if (tj <= ti) {
      for (int kk = 0; kk < DK; kk += 4) {
        float4 kj[4], ki[4], qi[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          kj[a] = *reinterpret_cast<const float4*>(sk + (4 * tj + a) * KP + kk);
          ki[a] = *reinterpret_cast<const float4*>(sk + (4 * ti + a) * KP + kk);
          qi[a] = *reinterpret_cast<const float4*>(sq + (4 * ti + a) * KP + kk);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
          for (int b2 = 0; b2 < 4; ++b2) {
            akk[a][b2] += ki[a].x * kj[b2].x + ki[a].y * kj[b2].y + ki[a].z * kj[b2].z + ki[a].w * kj[b2].w;
            aqk[a][b2] += qi[a].x * kj[b2].x + qi[a].y * kj[b2].y + qi[a].z * kj[b2].z + qi[a].w * kj[b2].w;
          }
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = 4 * ti + a;
      float aq_row[4];
#pragma unroll
      for (int b2 = 0; b2 < 4; ++b2) {
        const int j = 4 * tj + b2;
        const float dec = (j <= i) ? __expf(sgc[i] - sgc[j]) : 0.f;
        sA[i * AP + j] = (j < i) ? -sbeta[i] * akk[a][b2] * dec : 0.f;
        aq_row[b2] = (j <= i) ? aqk[a][b2] * dec : 0.f;
      }
      __half2 h01 = __floats2half2_rn(aq_row[0], aq_row[1]), h23 = __floats2half2_rn(aq_row[2], aq_row[3]);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&h01);
      pk.y = *reinterpret_cast<uint32_t*>(&h23);
      *reinterpret_cast<uint2*>(o.Aqk + ((size_t)(t0 + i) * Hv + h) * C + 4 * tj) = pk;
    }
  }
  __syncthreads();

  // forward substitution: row i <- row i + row i * A[:i, :i]   (warp 0, lanes own columns j and j+32)
  if (warp == 0) {
    for (int i = 1; i < C; ++i) {
      float n0 = 0.f, n1 = 0.f;
      const float* Ai = sA + i * AP;
      for (int m = 0; m < i; ++m) {
        const float aim = Ai[m];
        n0 += aim * sA[m * AP + lane];
        n1 += aim * sA[m * AP + 32 + lane];
      }
      __syncwarp();
      if (lane < i) sA[i * AP + lane] += n0;
      if (32 + lane < i) sA[i * AP + 32 + lane] += n1;
      __syncwarp();
    }
  }
  __syncthreads();

  // U = T (beta v), W = T (beta e^gc k), T = A + I; thread -> 8 rows x 4 cols, warp == row group
  {
    const int ri = tid >> 5, cj = tid & 31;
    float u[8][4], w[8][4];
#pragma unroll
    for (int a = 0; a < 8; ++a)
#pragma unroll
      for (int b2 = 0; b2 < 4; ++b2) u[a][b2] = w[a][b2] = 0.f;
    const int jmax = 8 * ri + 7;
    for (int j = 0; j <= jmax; ++j) {
      const float bj = sbeta[j];
      const float cw = bj * __expf(sgc[j]);
      const float4 kj = *reinterpret_cast<const float4*>(sk + j * KP + 4 * cj);
      const uint2 vu = *reinterpret_cast<const uint2*>(sv + j * DV + 4 * cj);
      const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vu);
      const float2 va = __bfloat1622float2(v2[0]), vb = __bfloat1622float2(v2[1]);
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        const int i = 8 * ri + a;
        const float tij = (j == i) ? 1.f : ((j < i) ? sA[i * AP + j] : 0.f);
        const float tu = tij * bj, tw = tij * cw;
        u[a][0] += tu * va.x; u[a][1] += tu * va.y; u[a][2] += tu * vb.x; u[a][3] += tu * vb.y;
        w[a][0] += tw * kj.x; w[a][1] += tw * kj.y; w[a][2] += tw * kj.z; w[a][3] += tw * kj.w;
      }
    }
    const float gl = sgc[C - 1];
    auto pack4 = [](float a, float b, float c2, float d) {
      __half2 x = __floats2half2_rn(a, b), y = __floats2half2_rn(c2, d);
      uint2 pk;
      pk.x = *reinterpret_cast<uint32_t*>(&x);
      pk.y = *reinterpret_cast<uint32_t*>(&y);
      return pk;
    };
    float kg[8][4];
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int i = 8 * ri + a;
      const size_t base = ((size_t)(t0 + i) * Hv + h) * DK + 4 * cj;
      *reinterpret_cast<float4*>(o.U + base) = make_float4(u[a][0], u[a][1], u[a][2], u[a][3]);
      *reinterpret_cast<uint2*>(o.W + base) = pack4(w[a][0], w[a][1], w[a][2], w[a][3]);
      const float eg = __expf(sgc[i]);
      const float ek = __expf(gl - sgc[i]);
      const float4 qv = *reinterpret_cast<const float4*>(sq + i * KP + 4 * cj);
      const float4 kv = *reinterpret_cast<const float4*>(sk + i * KP + 4 * cj);
      *reinterpret_cast<uint2*>(o.Qg + base) = pack4(qv.x * eg, qv.y * eg, qv.z * eg, qv.w * eg);
      kg[a][0] = kv.x * ek; kg[a][1] = kv.y * ek; kg[a][2] = kv.z * ek; kg[a][3] = kv.w * ek;
    }
    // transposed store: for key dim d the 8 tokens of this row group are contiguous (16 bytes)
#pragma unroll
    for (int d = 0; d < 4; ++d) {
      uint4 pk;
      __half2 p0 = __floats2half2_rn(kg[0][d], kg[1][d]), p1 = __floats2half2_rn(kg[2][d], kg[3][d]);
      __half2 p2 = __floats2half2_rn(kg[4][d], kg[5][d]), p3 = __floats2half2_rn(kg[6][d], kg[7][d]);
      pk.x = *reinterpret_cast<uint32_t*>(&p0); pk.y = *reinterpret_cast<uint32_t*>(&p1);
      pk.z = *reinterpret_cast<uint32_t*>(&p2); pk.w = *reinterpret_cast<uint32_t*>(&p3);
      *reinterpret_cast<uint4*>(o.KgT + (((size_t)c * Hv + h) * DK + 4 * cj + d) * C + 8 * ri) = pk;
    }
    if (tid == 0) o.Gl[(size_t)c * Hv + h] = __expf(gl);
  }
}

__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst_smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_1() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

// A fragment (16 rows x 16 k) of a row-major fp16 tile with row stride `ld` halves.
__device__ __forceinline__ void load_a(uint32_t (&a)[4], const __half* tile, int ld, int row0, int k0, int g, int tig) {
  const __half* p = tile + (size_t)(row0 + g) * ld + k0 + 2 * tig;
  a[0] = *reinterpret_cast<const uint32_t*>(p);
  a[1] = *reinterpret_cast<const uint32_t*>(p + 8 * ld);
  a[2] = *reinterpret_cast<const uint32_t*>(p + 8);
  a[3] = *reinterpret_cast<const uint32_t*>(p + 8 * ld + 8);
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Tensor-core form of gdn_prepare_kernel: the four products of a chunk (k k^T, q k^T, T (beta v), T (beta e^gc k)) run
// as m16n8k16 MMAs on fp16 copies of the normalised rows; the triangular inverse stays scalar fp32 but runs by blocks
// of 16 over the whole CTA.  Shared memory: three [64 x 128] fp16 tiles (k_hat, q_hat, v), the fp32 triangular
// matrix; the inverse and the two fp16 T tiles reuse the q_hat tile and the triangular matrix once those are dead,
// which keeps three CTAs on an SM.
constexpr int LDH = 136;  // padded row (halves) of the [64 x 128] tiles: fragment loads hit 32 distinct banks
constexpr int TSH = 72;   // padded row (halves) of the [64 x 64] T tiles
constexpr int PREP_MMA_SMEM = 3 * C * LDH * 2 + C * AP * 4 + 2 * C * 4;

__global__ void __launch_bounds__(256, 3)
gdn_prepare_mma_kernel(const __nv_bfloat16* __restrict__ mixed, int ld, int q_off, int k_off, int v_off,
                       const float* __restrict__ g, const float* __restrict__ beta, PrepOut o, int T, int Hv, int Hk,
                       float q_scale) {
  extern __shared__ __align__(16) unsigned char prep_raw[];
  __half* sKh = reinterpret_cast<__half*>(prep_raw);   // [64][LDH] k_hat
  __half* sQh = sKh + C * LDH;                         // [64][LDH] q_hat * scale
  __half* sVh = sQh + C * LDH;                         // [64][LDH] v
  float* sA = reinterpret_cast<float*>(sVh + C * LDH); // [64][AP]  T - I (strictly lower triangular)
  float* sgc = sA + C * AP;                            // [64] cumulative log decay
  float* sbeta = sgc + C;                              // [64]
  __half* sTb = reinterpret_cast<__half*>(sA);         // [64][TSH] T diag(beta)            (after the inversion)
  __half* sTw = sQh;                                   // [64][TSH] T diag(beta e^gc)       (after the inversion)
  const int h = blockIdx.x, c = blockIdx.y;
  const int kh = h / (Hv / Hk);
  const int t0 = c * C;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tig = lane & 3;

  if (warp == 0) {
    const int ta = t0 + lane, tb = t0 + 32 + lane;
    float ga = ta < T ? g[(size_t)ta * Hv + h] : 0.f;
    float gb = tb < T ? g[(size_t)tb * Hv + h] : 0.f;
#pragma unroll
    for (int ofs = 1; ofs < 32; ofs <<= 1) {
      const float x = __shfl_up_sync(0xffffffffu, ga, ofs);
      const float y = __shfl_up_sync(0xffffffffu, gb, ofs);
      if (lane >= ofs) { ga += x; gb += y; }
    }
    gb += __shfl_sync(0xffffffffu, ga, 31);
    sgc[lane] = ga;
    sgc[32 + lane] = gb;
    sbeta[lane] = ta < T ? beta[(size_t)ta * Hv + h] : 0.f;
    sbeta[32 + lane] = tb < T ? beta[(size_t)tb * Hv + h] : 0.f;
  }
  __syncthreads();

  // rows: normalise, keep fp16 copies, write q_hat e^gc
  for (int r = warp; r < C; r += 8) {
    const int t = t0 + r;
    float kf[4] = {0, 0, 0, 0}, qf[4] = {0, 0, 0, 0}, vf[4] = {0, 0, 0, 0};
    if (t < T) {
      const __nv_bfloat16* row = mixed + (size_t)t * ld;
      const uint2 ku = *reinterpret_cast<const uint2*>(row + k_off + kh * DK + lane * 4);
      const uint2 qu = *reinterpret_cast<const uint2*>(row + q_off + kh * DK + lane * 4);
      const uint2 vu = *reinterpret_cast<const uint2*>(row + v_off + h * DV + lane * 4);
      const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&ku);
      const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&qu);
      const __nv_bfloat162* v2 = reinterpret_cast<const __nv_bfloat162*>(&vu);
      float2 a = __bfloat1622float2(k2[0]), bb = __bfloat1622float2(k2[1]);
      kf[0] = a.x; kf[1] = a.y; kf[2] = bb.x; kf[3] = bb.y;
      a = __bfloat1622float2(q2[0]); bb = __bfloat1622float2(q2[1]);
      qf[0] = a.x; qf[1] = a.y; qf[2] = bb.x; qf[3] = bb.y;
      a = __bfloat1622float2(v2[0]); bb = __bfloat1622float2(v2[1]);
      vf[0] = a.x; vf[1] = a.y; vf[2] = bb.x; vf[3] = bb.y;
    }
    const float kn = rsqrtf(warp_sum(kf[0] * kf[0] + kf[1] * kf[1] + kf[2] * kf[2] + kf[3] * kf[3]) + 1e-6f);
    const float qn = rsqrtf(warp_sum(qf[0] * qf[0] + qf[1] * qf[1] + qf[2] * qf[2] + qf[3] * qf[3]) + 1e-6f) * q_scale;
    uint2 pk;
    pk.x = pack_h2(kf[0] * kn, kf[1] * kn); pk.y = pack_h2(kf[2] * kn, kf[3] * kn);
    *reinterpret_cast<uint2*>(sKh + r * LDH + lane * 4) = pk;
    pk.x = pack_h2(qf[0] * qn, qf[1] * qn); pk.y = pack_h2(qf[2] * qn, qf[3] * qn);
    *reinterpret_cast<uint2*>(sQh + r * LDH + lane * 4) = pk;
    pk.x = pack_h2(vf[0], vf[1]); pk.y = pack_h2(vf[2], vf[3]);
    *reinterpret_cast<uint2*>(sVh + r * LDH + lane * 4) = pk;
    const float eg = __expf(sgc[r]) * qn;
    pk.x = pack_h2(qf[0] * eg, qf[1] * eg); pk.y = pack_h2(qf[2] * eg, qf[3] * eg);
    *reinterpret_cast<uint2*>(o.Qg + ((size_t)(t0 + r) * Hv + h) * DK + lane * 4) = pk;
  }
  __syncthreads();

  // k k^T and q k^T: warp -> rows [16 mt, 16 mt + 16) x columns [32 nh, 32 nh + 32); tiles above the diagonal are skipped
  {
    const int mt = warp & 3, nh = warp >> 2;
    const int last = 16 * mt + 15 - 32 * nh;                 // largest useful column offset inside this warp's half
    const int ntiles = last < 0 ? 0 : min(4, last / 8 + 1);
    float akk[4][4], aqk[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) akk[n][e] = aqk[n][e] = 0.f;
    if (ntiles > 0) {
#pragma unroll 2
      for (int ks = 0; ks < DK / 16; ++ks) {
        uint32_t ak[4], aq[4];
        load_a(ak, sKh, LDH, 16 * mt, 16 * ks, gq, tig);
        load_a(aq, sQh, LDH, 16 * mt, 16 * ks, gq, tig);
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          if (n < ntiles) {
            const __half* bp = sKh + (size_t)(32 * nh + 8 * n + gq) * LDH + 16 * ks + 2 * tig;
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(bp), b1 = *reinterpret_cast<const uint32_t*>(bp + 8);
            mma16816(akk[n], ak, b0, b1);
            mma16816(aqk[n], aq, b0, b1);
          }
        }
      }
    }
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int i = 16 * mt + gq + 8 * hf, j = 32 * nh + 8 * n + 2 * tig;
        const float gi = sgc[i], bi = sbeta[i];
        float av[2], qv[2];
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const int jj = j + e;
          const float dec = (jj <= i) ? __expf(gi - sgc[jj]) : 0.f;
          av[e] = (jj < i) ? -bi * akk[n][2 * hf + e] * dec : 0.f;
          qv[e] = (jj <= i) ? aqk[n][2 * hf + e] * dec : 0.f;
        }
        sA[i * AP + j] = av[0];
        sA[i * AP + j + 1] = av[1];
        *reinterpret_cast<uint32_t*>(o.Aqk + ((size_t)(t0 + i) * Hv + h) * C + j) = pack_h2(qv[0], qv[1]);
      }
  }
  __syncthreads();

  // T = (I - A)^-1 by blocks of 16 (A strictly lower triangular, fp32):
  //   T_ii = (I - A_ii)^-1                       four warps, one diagonal block each, rows in registers
  //   T_ij = T_ii (sum_{k=j}^{i-1} A_ik T_kj)    one block sub-diagonal at a time, every thread one element per block
  // T is built in sX (the dead q_hat tile); the inner sums are staged in the unused upper blocks of sA.
  float* sX = reinterpret_cast<float*>(sQh);                  // [64][AP]
  if (warp < 4) {
    if (lane < 16) {
      const int b0 = 16 * warp;
      float tr[16];
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        float acc = (lane == r) ? 1.f : 0.f;
#pragma unroll
        for (int m = 0; m < r; ++m) acc += sA[(b0 + r) * AP + b0 + m] * tr[m];
        tr[r] = acc;
        sX[(b0 + r) * AP + b0 + lane] = acc;
      }
    }
  } else {
    // blocks above the diagonal are zero: (0,1) (0,2) (0,3) (1,2) (1,3) (2,3)
    for (int e = (warp - 4) * 32 + lane; e < 6 * 256; e += 128) {
      const int blk = e >> 8, r = (e >> 4) & 15, cc = e & 15;
      const int bi = blk < 3 ? 0 : (blk < 5 ? 1 : 2);
      const int bj = blk < 3 ? blk + 1 : (blk < 5 ? blk - 1 : 3);
      sX[(16 * bi + r) * AP + 16 * bj + cc] = 0.f;
    }
  }
  __syncthreads();
  {
    const int r = tid >> 4, cc = tid & 15;
#pragma unroll 1
    for (int d = 1; d < 4; ++d) {
      float mv[3];
      for (int b = 0; b + d < 4; ++b) {                       // block (i, j) = (b + d, b)
        const int bi = b + d, bj = b;
        float acc = 0.f;
        for (int k = bj; k < bi; ++k) {
          const float* ar = sA + (16 * bi + r) * AP + 16 * k;
          const float* xc = sX + (16 * k) * AP + 16 * bj + cc;
#pragma unroll
          for (int m = 0; m < 16; ++m) acc += ar[m] * xc[m * AP];
        }
        mv[b] = acc;
      }
      for (int b = 0; b + d < 4; ++b) sA[(16 * b + r) * AP + 16 * (b + d) + cc] = mv[b];     // staged at (j, i)
      __syncthreads();
      for (int b = 0; b + d < 4; ++b) {
        const int bi = b + d, bj = b;
        const float* tr = sX + (16 * bi + r) * AP + 16 * bi;
        const float* mc = sA + (16 * bj) * AP + 16 * bi + cc;
        float acc = 0.f;
#pragma unroll
        for (int m = 0; m < 16; ++m) acc += tr[m] * mc[m * AP];
        sX[(16 * bi + r) * AP + 16 * bj + cc] = acc;
      }
      __syncthreads();
    }
  }

  // T as fp16 A operands with beta (and e^gc) folded into the columns: sTb takes the place of A, sTw that of T
  {
    const int i = tid >> 2, j0 = (tid & 3) * 16;
    float tv[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) tv[e] = sX[i * AP + j0 + e];
    __syncthreads();                                          // every read of sX is done before sTw overwrites it
#pragma unroll
    for (int e = 0; e < 16; e += 2) {
      const float b0 = sbeta[j0 + e], b1 = sbeta[j0 + e + 1];
      *reinterpret_cast<uint32_t*>(sTb + i * TSH + j0 + e) = pack_h2(tv[e] * b0, tv[e + 1] * b1);
      *reinterpret_cast<uint32_t*>(sTw + i * TSH + j0 + e) =
          pack_h2(tv[e] * b0 * __expf(sgc[j0 + e]), tv[e + 1] * b1 * __expf(sgc[j0 + e + 1]));
    }
  }
  __syncthreads();

  // W = Tw k_hat and U = Tb v: warp -> rows [16 mt, +16) x columns [64 nh, +64); k-steps past the diagonal are zero
  {
    const int mt = warp & 3, nh = warp >> 2;
#pragma unroll 1
    for (int which = 0; which < 2; ++which) {
      const __half* tA = which ? sTb : sTw;
      const __half* tB = which ? sVh : sKh;
      float acc[8][4];
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;
      for (int kk = 0; kk <= mt; ++kk) {
        uint32_t a[4];
        load_a(a, tA, TSH, 16 * mt, 16 * kk, gq, tig);
#pragma unroll
        for (int n = 0; n < 8; n += 2) {
          uint32_t b[4];
          ldmatrix_x4_trans(b, tB + (size_t)(16 * kk + (lane & 7) + ((lane >> 3) & 1) * 8) * LDH + 64 * nh + (n + (lane >> 4)) * 8);
          mma16816(acc[n], a, b[0], b[1]);
          mma16816(acc[n + 1], a, b[2], b[3]);
        }
      }
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          const int i = 16 * mt + gq + 8 * hf, col = 64 * nh + 8 * n + 2 * tig;
          const size_t base = ((size_t)(t0 + i) * Hv + h) * DK + col;
          if (which) *reinterpret_cast<float2*>(o.U + base) = make_float2(acc[n][2 * hf], acc[n][2 * hf + 1]);
          else *reinterpret_cast<uint32_t*>(o.W + base) = pack_h2(acc[n][2 * hf], acc[n][2 * hf + 1]);
        }
    }
  }

  // (k_hat e^(gc_last - gc))^T: key dim major, eight tokens (16 bytes) per store, eight lanes cover one key dim's row
  {
    const float gl = sgc[C - 1];
    const int seg = tid & 7;
    float ek[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) ek[e] = __expf(gl - sgc[8 * seg + e]);
    for (int d = tid >> 3; d < DK; d += 32) {
      float kv[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) kv[e] = __half2float(sKh[(8 * seg + e) * LDH + d]) * ek[e];
      uint4 pk;
      pk.x = pack_h2(kv[0], kv[1]); pk.y = pack_h2(kv[2], kv[3]); pk.z = pack_h2(kv[4], kv[5]); pk.w = pack_h2(kv[6], kv[7]);
      *reinterpret_cast<uint4*>(o.KgT + (((size_t)c * Hv + h) * DK + d) * C + 8 * seg) = pk;
    }
    if (tid == 0) o.Gl[(size_t)c * Hv + h] = __expf(gl);
  }
}
// ------------------------------------------------------------ inter-chunk scan
constexpr int SL = 32;    // value columns per CTA
constexpr int WS = 136;   // padded row (halves) of the [64 x 128] W / Qg tiles and of the [32 x 128] state copy
constexpr int TS = 72;    // padded row (halves) of the [. x 64] tiles (KgT, Aqk, v_new^T)
constexpr int SCAN_WQ_HALVES = 2 * C * WS;                                // W, Qg of one chunk (double-buffered)
constexpr int SCAN_KA_HALVES = DK * TS + C * TS;                          // KgT, Aqk of one chunk (single buffer)
// 110.6 KB: two CTAs per SM, so that 4 x 48 heads run as one wave and one CTA's waits overlap the other's MMAs
constexpr int SCAN_SMEM_BYTES = (2 * SCAN_WQ_HALVES + SCAN_KA_HALVES + SL * WS + SL * TS) * 2;

// grid (Hv, 128 / SL), 128 threads.  Warp w owns tokens [16w, 16w+16) of the chunk for v_new and O, and state rows
// (key dims) [32w, 32w+32) for the state update.
__global__ void __launch_bounds__(128, 2)
gdn_scan_kernel(PrepOut w, float* __restrict__ state, __nv_bfloat16* __restrict__ out, int T, int nchunks, int Hv) {
  extern __shared__ __align__(16) __half sh[];
  __half* const bK = sh + 2 * SCAN_WQ_HALVES;     // [128][TS] KgT of the current chunk
  __half* const bA = bK + DK * TS;                // [64][TS]  Aqk of the current chunk
  __half* sS = bA + C * TS;                // [SL][WS]  state^T operand copy: value column major, key dim minor
  __half* sV = sS + SL * WS;               // [SL][TS]  v_new^T: value column major, token minor
  const int h = blockIdx.x, sl = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
  float* Sg = state + (size_t)h * DK * DV + sl * SL;

  // W / Qg are needed at the top of a step and are fetched one chunk ahead; KgT / Aqk are needed after v_new and are
  // fetched at the top of their own step (their buffer is free once every warp has left the previous step)
  auto prefetch_wq = [&](int c) {
    __half* bW = sh + (c & 1) * SCAN_WQ_HALVES, *bQ = bW + C * WS;
    const size_t t0 = (size_t)c * C;
    for (int i = tid; i < C * 16; i += 128) {            // 64 rows x 16 copies of 16 bytes
      const int r = i >> 4, q = i & 15;
      const size_t src = ((t0 + r) * Hv + h) * DK + q * 8;
      cp_async16(bW + r * WS + q * 8, w.W + src);
      cp_async16(bQ + r * WS + q * 8, w.Qg + src);
    }
    cp_async_commit();
  };
  auto prefetch_ka = [&](int c) {
    const size_t t0 = (size_t)c * C;
    for (int i = tid; i < DK * 8; i += 128) {            // 128 rows x 8 copies
      const int r = i >> 3, q = i & 7;
      cp_async16(bK + r * TS + q * 8, w.KgT + (((size_t)c * Hv + h) * DK + r) * C + q * 8);
    }
    for (int i = tid; i < C * 8; i += 128) {
      const int r = i >> 3, q = i & 7;
      cp_async16(bA + r * TS + q * 8, w.Aqk + ((t0 + r) * Hv + h) * C + q * 8);
    }
    cp_async_commit();
  };

  // state rows 32w + 16mt + g (+8), columns 8nt + 2tig (+1), in accumulator-fragment order
  float sacc[2][4][4];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = 32 * warp + 16 * mt + g + (e >> 1) * 8, n = 8 * nt + 2 * tig + (e & 1);
        const float v = Sg[(size_t)m * DV + n];
        sacc[mt][nt][e] = v;
        sS[n * WS + m] = __float2half_rn(v);
      }
  prefetch_wq(0);

  // U rows of this thread and the chunk's decay are plain global loads on the serial chain: both are fetched one
  // chunk ahead (into registers) so that their latency is paid under the previous chunk's MMAs
  auto load_u = [&](int c, float2 (&dst)[4][2]) {
    const int t0 = c * C;
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf)
        dst[nt][hf] = *reinterpret_cast<const float2*>(w.U + ((size_t)(t0 + 16 * warp + g + 8 * hf) * Hv + h) * DV +
                                                        sl * SL + 8 * nt + 2 * tig);
  };
  float2 u_next[4][2];
  load_u(0, u_next);
  float gl_next = w.Gl[h];

  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * C;
    cp_async_wait_all();
    __syncthreads();                       // W / Qg of chunk c landed; the state copy of chunk c-1 is complete; sV, bK, bA are free
    prefetch_ka(c);
    const bool more = c + 1 < nchunks;
    if (more) prefetch_wq(c + 1);
    const __half* bW = sh + (c & 1) * SCAN_WQ_HALVES, *bQ = bW + C * WS;

    float2 u[4][2];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) u[nt][hf] = u_next[nt][hf];
    const float gl = gl_next;
    if (more) {
      load_u(c + 1, u_next);
      gl_next = w.Gl[(size_t)(c + 1) * Hv + h];
    }
    // v_new = U - W S and O = Qg S read the same state operand: one pass over the key dim feeds both (eight
    // independent accumulator chains per warp, one shared-memory read of the state fragment for two MMAs)
    float accv[4][4], acc[4][4];
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) { accv[nt][e] = 0.f; acc[nt][e] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < DK / 16; ++ks) {
      uint32_t aw[4], aq[4];
      load_a(aw, bW, WS, 16 * warp, 16 * ks, g, tig);
      load_a(aq, bQ, WS, 16 * warp, 16 * ks, g, tig);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const __half* bp = sS + (8 * nt + g) * WS + 16 * ks + 2 * tig;
        const uint32_t s0 = *reinterpret_cast<const uint32_t*>(bp), s1 = *reinterpret_cast<const uint32_t*>(bp + 8);
        mma16816(accv[nt], aw, s0, s1);
        mma16816(acc[nt], aq, s0, s1);
      }
    }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt) {
      const int n = 8 * nt + 2 * tig, r = 16 * warp + g;
      sV[n * TS + r] = __float2half_rn(u[nt][0].x - accv[nt][0]);
      sV[(n + 1) * TS + r] = __float2half_rn(u[nt][0].y - accv[nt][1]);
      sV[n * TS + r + 8] = __float2half_rn(u[nt][1].x - accv[nt][2]);
      sV[(n + 1) * TS + r + 8] = __float2half_rn(u[nt][1].y - accv[nt][3]);
    }
    // S e^gl before the barrier: pure register work that overlaps the other warps' v_new
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) sacc[mt][nt][e] *= gl;
    if (more) cp_async_wait_1(); else cp_async_wait_all();   // this thread's KgT / Aqk copies (the older group) are done
    __syncthreads();                       // v_new^T, KgT, Aqk complete; every warp is done reading the old state copy
    // O += Aqk v_new and S += KgT v_new share the v_new^T operand: twelve independent chains over the chunk's tokens
#pragma unroll
    for (int ks = 0; ks < C / 16; ++ks) {
      uint32_t b0[4], b1[4];
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) {
        const __half* bp = sV + (8 * nt + g) * TS + 16 * ks + 2 * tig;
        b0[nt] = *reinterpret_cast<const uint32_t*>(bp);
        b1[nt] = *reinterpret_cast<const uint32_t*>(bp + 8);
      }
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) {
        uint32_t a[4];
        load_a(a, bK, TS, 32 * warp + 16 * mt, 16 * ks, g, tig);
#pragma unroll
        for (int nt = 0; nt < 4; ++nt) mma16816(sacc[mt][nt], a, b0[nt], b1[nt]);
      }
      uint32_t aa[4];
      load_a(aa, bA, TS, 16 * warp, 16 * ks, g, tig);
#pragma unroll
      for (int nt = 0; nt < 4; ++nt) mma16816(acc[nt], aa, b0[nt], b1[nt]);
    }
    // the next chunk starts from the fp16 copy of the new state: publish it first, store the outputs after
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < 4; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int m = 32 * warp + 16 * mt + g + (e >> 1) * 8, n = 8 * nt + 2 * tig + (e & 1);
          sS[n * WS + m] = __float2half_rn(sacc[mt][nt][e]);
        }
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int t = t0 + 16 * warp + g + 8 * hf;
        if (t < T)
          *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * Hv + h) * DV + sl * SL + 8 * nt + 2 * tig) =
              __floats2bfloat162_rn(acc[nt][2 * hf], acc[nt][2 * hf + 1]);
      }
  }
#pragma unroll
  for (int mt = 0; mt < 2; ++mt)
#pragma unroll
    for (int nt = 0; nt < 4; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int m = 32 * warp + 16 * mt + g + (e >> 1) * 8, n = 8 * nt + 2 * tig + (e & 1);
        Sg[(size_t)m * DV + n] = sacc[mt][nt][e];
      }
}

}  // namespace

static int g_prepare_simt = 0;

extern "C" {

// 1: run the chunk preparation with the scalar fp32 kernel (kept as the numerical yardstick of the tensor-core one).
int b200_gdn_use_simt_prepare(int on) {
  const int was = g_prepare_simt;
  g_prepare_simt = on ? 1 : 0;
  return was;
}

// Floats of workspace needed by b200_gdn_chunked for T tokens and Hv value heads.
long long b200_gdn_workspace_floats(int T, int Hv) {
  const long long nch = (T + C - 1) / C;
  const long long Tp = nch * C;
  // U fp32 [Tp,Hv,128]; W, Qg, KgT fp16 [Tp,Hv,128] each; Aqk fp16 [Tp,Hv,64]; Gl fp32 [nch,Hv]
  return Tp * Hv * (128LL + 3 * 64 + 32) + nch * Hv;
}

// mixed: [T, ld] bf16 holding q (Hk*128 at q_off), k (k_off) and v (Hv*128 at v_off) after conv+SiLU.
// g, beta: [T, Hv] fp32. state: [Hv, 128, 128] fp32, updated in place. out: [T, Hv, 128] bf16.
int b200_gdn_chunked(const void* mixed, int ld, int q_off, int k_off, int v_off, const float* g, const float* beta,
                     float* state, void* out, float* workspace, int T, int Hv, int Hk, cudaStream_t stream) {
  if (T <= 0 || Hv % Hk) return -6;
  const int nch = (T + C - 1) / C;
  const size_t Tp = (size_t)nch * C;
  PrepOut o;
  o.U = workspace;
  o.W = reinterpret_cast<__half*>(o.U + Tp * Hv * 128);
  o.Qg = o.W + Tp * Hv * 128;
  o.KgT = o.Qg + Tp * Hv * 128;
  o.Aqk = o.KgT + Tp * Hv * 128;
  o.Gl = reinterpret_cast<float*>(o.Aqk + Tp * Hv * 64);
  const float q_scale = 0.08838834764831845f;  // 1/sqrt(128)
  const int prep_smem = (2 * C * KP + C * AP + 2 * C) * 4 + C * DV * 2;
  const int scan_smem = SCAN_SMEM_BYTES;
  static b200::PerDeviceOnce once_;
  bool& configured = once_.slot();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, prep_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gdn_prepare_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PREP_MMA_SMEM);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gdn_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, scan_smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (g_prepare_simt)
    gdn_prepare_kernel<<<dim3(Hv, nch), 256, prep_smem, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(mixed), ld, q_off, k_off, v_off, g, beta, o, T, Hv, Hk, q_scale);
  else
    gdn_prepare_mma_kernel<<<dim3(Hv, nch), 256, PREP_MMA_SMEM, stream>>>(
        reinterpret_cast<const __nv_bfloat16*>(mixed), ld, q_off, k_off, v_off, g, beta, o, T, Hv, Hk, q_scale);
  gdn_scan_kernel<<<dim3(Hv, DV / SL), 128, scan_smem, stream>>>(o, state, reinterpret_cast<__nv_bfloat16*>(out), T,
                                                                  nch, Hv);
  return (int)cudaGetLastError();
}

// One token per sequence: mixed [B, ld], g/beta [B, Hv], states [slots, Hv, 128, 128], out [B, Hv, 128].
int b200_gdn_step(float* states, long long slot_stride, const int* slot_ids, const void* mixed, int ld, int q_off,
                  int k_off, int v_off, const float* g, const float* beta, void* out, int B, int Hv, int Hk,
                  cudaStream_t stream) {
  if (B <= 0 || Hv % Hk) return -6;
  gdn_step_kernel<<<dim3(Hv, B), 128, 0, stream>>>(states, (size_t)slot_stride, slot_ids,
                                                    reinterpret_cast<const __nv_bfloat16*>(mixed), ld, q_off, k_off,
                                                    v_off, g, beta, reinterpret_cast<__nv_bfloat16*>(out), Hv, Hk,
                                                    0.08838834764831845f);
  return (int)cudaGetLastError();
}

}  // extern "C"
