// Gated DeltaNet (gated delta rule) for head dims dk = dv = 128:
//   * gdn_step    - single-token recurrence for decode batches (one state per slot);
//   * gdn_prepare - chunk-parallel part of the chunked scan (chunk 64): L2-normalised
//                   q/k, in-chunk cumulative log-decay, the (I - A)^-1 "UT transform"
//                   by forward substitution, U = T (beta v), W = T (beta e^gc k),
//                   and the decayed q k^T block;
//   * gdn_scan    - the sequential inter-chunk recurrence, one CTA per (head, 32-wide
//                   value slice): v_new = U - W S, O = (q e^gc) S + Aqk v_new,
//                   S = S e^gc_last + (k e^(gc_last-gc))^T v_new, state kept in shared
//                   memory in fp32 across all chunks of the call.
// The chunked form is algebraically the recurrence
//   S_t = e^{g_t} S_{t-1} + k_t (beta_t (v_t - (e^{g_t} S_{t-1})^T k_t))^T,  o_t = S_t^T q_t / sqrt(dk)
// and replaces the reference's per-token serial kernels
// (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:2282-2600, qwen_gdn_flashqla.cu:36);
// the math oracle is the chunked PyTorch form src/models/qwen4_exp/attention.py:184-270.
#include <cuda_bf16.h>
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
struct PrepOut {
  float* U;    // [Tp, Hv, 128]  T (beta v)
  float* W;    // [Tp, Hv, 128]  T (beta e^gc k)
  float* Qg;   // [Tp, Hv, 128]  q_hat * scale * e^gc
  float* Kg;   // [Tp, Hv, 128]  k_hat * e^(gc_last - gc)
  float* Aqk;  // [Tp, Hv, 64]   (q_hat*scale . k_hat) e^(gc_i - gc_j), j <= i
  float* Gl;   // [nchunks, Hv]  e^gc_last
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
      *reinterpret_cast<float4*>(o.Aqk + ((size_t)(t0 + i) * Hv + h) * C + 4 * tj) =
          make_float4(aq_row[0], aq_row[1], aq_row[2], aq_row[3]);
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
#pragma unroll
    for (int a = 0; a < 8; ++a) {
      const int i = 8 * ri + a;
      const size_t base = ((size_t)(t0 + i) * Hv + h) * DK + 4 * cj;
      *reinterpret_cast<float4*>(o.U + base) = make_float4(u[a][0], u[a][1], u[a][2], u[a][3]);
      *reinterpret_cast<float4*>(o.W + base) = make_float4(w[a][0], w[a][1], w[a][2], w[a][3]);
      const float eg = __expf(sgc[i]);
      const float ek = __expf(gl - sgc[i]);
      const float4 qv = *reinterpret_cast<const float4*>(sq + i * KP + 4 * cj);
      const float4 kv = *reinterpret_cast<const float4*>(sk + i * KP + 4 * cj);
      *reinterpret_cast<float4*>(o.Qg + base) = make_float4(qv.x * eg, qv.y * eg, qv.z * eg, qv.w * eg);
      *reinterpret_cast<float4*>(o.Kg + base) = make_float4(kv.x * ek, kv.y * ek, kv.z * ek, kv.w * ek);
    }
    if (tid == 0) o.Gl[(size_t)c * Hv + h] = __expf(gl);
  }
}

// ------------------------------------------------------------ inter-chunk scan
constexpr int SL = 32;  // value columns per CTA
__global__ void __launch_bounds__(256, 1)
gdn_scan_kernel(PrepOut w, float* __restrict__ state, __nv_bfloat16* __restrict__ out, int T, int nchunks, int Hv) {
  extern __shared__ float sm[];
  float* sW = sm;                 // [64][KP]
  float* sQ = sW + C * KP;        // [64][KP]
  float* sK = sQ + C * KP;        // [64][KP]
  float* sAq = sK + C * KP;       // [64][AP]
  float* sS = sAq + C * AP;       // [128][SL]
  float* sVn = sS + DK * SL;      // [64][SL]
  const int h = blockIdx.x, sl = blockIdx.y;
  const int tid = threadIdx.x;
  float* Sg = state + (size_t)h * DK * DV + sl * SL;
  for (int i = tid; i < DK * SL; i += 256) sS[i] = Sg[(size_t)(i / SL) * DV + (i % SL)];

  const int rg = tid >> 4, cg = tid & 15;  // 4 rows x 2 cols for [64 x 32] products
  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * C;
    __syncthreads();
    for (int i = tid; i < C * (DK / 4); i += 256) {
      const int r = i / (DK / 4), q4 = i % (DK / 4);
      const size_t base = ((size_t)(t0 + r) * Hv + h) * DK + q4 * 4;
      *reinterpret_cast<float4*>(sW + r * KP + q4 * 4) = *reinterpret_cast<const float4*>(w.W + base);
      *reinterpret_cast<float4*>(sQ + r * KP + q4 * 4) = *reinterpret_cast<const float4*>(w.Qg + base);
      *reinterpret_cast<float4*>(sK + r * KP + q4 * 4) = *reinterpret_cast<const float4*>(w.Kg + base);
    }
    for (int i = tid; i < C * C; i += 256) sAq[(i / C) * AP + (i % C)] = w.Aqk[((size_t)(t0 + i / C) * Hv + h) * C + (i % C)];
    __syncthreads();
    // v_new = U - W S
    float acc[4][2];
#pragma unroll
    for (int a = 0; a < 4; ++a) acc[a][0] = acc[a][1] = 0.f;
    for (int k = 0; k < DK; k += 4) {
      float4 wv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) wv[a] = *reinterpret_cast<const float4*>(sW + (4 * rg + a) * KP + k);
      const float2 s0 = *reinterpret_cast<const float2*>(sS + (k + 0) * SL + 2 * cg);
      const float2 s1 = *reinterpret_cast<const float2*>(sS + (k + 1) * SL + 2 * cg);
      const float2 s2 = *reinterpret_cast<const float2*>(sS + (k + 2) * SL + 2 * cg);
      const float2 s3 = *reinterpret_cast<const float2*>(sS + (k + 3) * SL + 2 * cg);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        acc[a][0] += wv[a].x * s0.x + wv[a].y * s1.x + wv[a].z * s2.x + wv[a].w * s3.x;
        acc[a][1] += wv[a].x * s0.y + wv[a].y * s1.y + wv[a].z * s2.y + wv[a].w * s3.y;
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int r = 4 * rg + a;
      const float2 u = *reinterpret_cast<const float2*>(w.U + ((size_t)(t0 + r) * Hv + h) * DV + sl * SL + 2 * cg);
      sVn[r * SL + 2 * cg] = u.x - acc[a][0];
      sVn[r * SL + 2 * cg + 1] = u.y - acc[a][1];
    }
    __syncthreads();
    // O = Qg S + Aqk v_new
#pragma unroll
    for (int a = 0; a < 4; ++a) acc[a][0] = acc[a][1] = 0.f;
    for (int k = 0; k < DK; k += 4) {
      float4 qv[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) qv[a] = *reinterpret_cast<const float4*>(sQ + (4 * rg + a) * KP + k);
      const float2 s0 = *reinterpret_cast<const float2*>(sS + (k + 0) * SL + 2 * cg);
      const float2 s1 = *reinterpret_cast<const float2*>(sS + (k + 1) * SL + 2 * cg);
      const float2 s2 = *reinterpret_cast<const float2*>(sS + (k + 2) * SL + 2 * cg);
      const float2 s3 = *reinterpret_cast<const float2*>(sS + (k + 3) * SL + 2 * cg);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        acc[a][0] += qv[a].x * s0.x + qv[a].y * s1.x + qv[a].z * s2.x + qv[a].w * s3.x;
        acc[a][1] += qv[a].x * s0.y + qv[a].y * s1.y + qv[a].z * s2.y + qv[a].w * s3.y;
      }
    }
    for (int j = 0; j < C; ++j) {
      const float2 vn = *reinterpret_cast<const float2*>(sVn + j * SL + 2 * cg);
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float aq = sAq[(4 * rg + a) * AP + j];
        acc[a][0] += aq * vn.x;
        acc[a][1] += aq * vn.y;
      }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int t = t0 + 4 * rg + a;
      if (t < T) {
        __nv_bfloat162 ob = __floats2bfloat162_rn(acc[a][0], acc[a][1]);
        *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)t * Hv + h) * DV + sl * SL + 2 * cg) = ob;
      }
    }
    __syncthreads();
    // S = S e^gl + Kg^T v_new : thread -> 8 state rows x 2 cols
    {
      const float gl = w.Gl[(size_t)c * Hv + h];
      float sacc[8][2];
#pragma unroll
      for (int a = 0; a < 8; ++a) {
        const float2 s = *reinterpret_cast<const float2*>(sS + (8 * rg + a) * SL + 2 * cg);
        sacc[a][0] = s.x * gl;
        sacc[a][1] = s.y * gl;
      }
      for (int r = 0; r < C; ++r) {
        const float2 vn = *reinterpret_cast<const float2*>(sVn + r * SL + 2 * cg);
        const float4 k0 = *reinterpret_cast<const float4*>(sK + r * KP + 8 * rg);
        const float4 k1 = *reinterpret_cast<const float4*>(sK + r * KP + 8 * rg + 4);
        const float kk[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w};
#pragma unroll
        for (int a = 0; a < 8; ++a) {
          sacc[a][0] += kk[a] * vn.x;
          sacc[a][1] += kk[a] * vn.y;
        }
      }
#pragma unroll
      for (int a = 0; a < 8; ++a)
        *reinterpret_cast<float2*>(sS + (8 * rg + a) * SL + 2 * cg) = make_float2(sacc[a][0], sacc[a][1]);
    }
  }
  __syncthreads();
  for (int i = tid; i < DK * SL; i += 256) Sg[(size_t)(i / SL) * DV + (i % SL)] = sS[i];
}

}  // namespace

extern "C" {

// Floats of workspace needed by b200_gdn_chunked for T tokens and Hv value heads.
long long b200_gdn_workspace_floats(int T, int Hv) {
  const long long nch = (T + C - 1) / C;
  const long long Tp = nch * C;
  return Tp * Hv * (4LL * 128 + 64) + nch * Hv;
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
  o.W = o.U + Tp * Hv * 128;
  o.Qg = o.W + Tp * Hv * 128;
  o.Kg = o.Qg + Tp * Hv * 128;
  o.Aqk = o.Kg + Tp * Hv * 128;
  o.Gl = o.Aqk + Tp * Hv * 64;
  const float q_scale = 0.08838834764831845f;  // 1/sqrt(128)
  const int prep_smem = (2 * C * KP + C * AP + 2 * C) * 4 + C * DV * 2;
  const int scan_smem = (3 * C * KP + C * AP + DK * SL + C * SL) * 4;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gdn_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, prep_smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gdn_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, scan_smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  gdn_prepare_kernel<<<dim3(Hv, nch), 256, prep_smem, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(mixed), ld, q_off, k_off, v_off, g, beta, o, T, Hv, Hk, q_scale);
  gdn_scan_kernel<<<dim3(Hv, DV / SL), 256, scan_smem, stream>>>(o, state, reinterpret_cast<__nv_bfloat16*>(out), T,
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
