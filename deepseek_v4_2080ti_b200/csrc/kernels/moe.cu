// Routed-expert plumbing around the grouped GEMM (gemm_wdec.cu, grouped mode):
//   moe_route        - scores (softmax | sigmoid | sqrt-softplus) + selection bias + top-k + weight normalisation;
//   moe_plan         - counting sort of the (token, k) routes by local expert: per-expert offsets, the row of every
//                      route in expert-sorted order, and the (expert, m_tile, row0, rows) work table of both grouped
//                      GEMMs, all on the device (nothing is read back by the host);
//   moe_gather       - token rows -> expert-sorted rows;
//   moe_swiglu       - silu(gate) * up on the sorted rows (with the DeepSeek clamp);
//   moe_combine      - out[t] = (shared[t]) + sum_k w[t,k] * y[row(t,k)], k ascending (deterministic).
// Routes whose expert lives on another rank are dropped locally (expert-range sharding) or carried by the
// dispatch kernels of csrc/comm.
// Reference counterparts: gate_topk_finalize (cpp_engine/backends/cuda/kernels/bf16_ops.cu:179-295),
// moe_route_count/prefix/fill (fp4_ops.cu:100-137), gather/scatter routes (src/csrc/cuda_kernel_impl.cu:264-331),
// moe_finalize_reduce (:4917).
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int MAX_TOPK = 16;
constexpr int MAX_EXPERTS = 1024;

__device__ __forceinline__ float score_fn(float x, int fn) {
  if (fn == 1) return 1.f / (1.f + __expf(-x));                       // sigmoid
  if (fn == 2) return sqrtf(x > 20.f ? x : log1pf(__expf(x)));        // sqrt(softplus)
  return x;                                                           // softmax handled by the caller
}

// One warp per token. logits fp32 [T, E]; bias fp32 [E] or null.
__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int K,
                                 int fn, int norm_topk, float route_scale, int* __restrict__ idx,
                                 float* __restrict__ wts) {
  const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const float* row = logits + (size_t)t * E;
  // softmax statistics
  float mx = -INFINITY, den = 1.f;
  if (fn == 0) {
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, row[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    den = 0.f;
    for (int e = lane; e < E; e += 32) den += __expf(row[e] - mx);
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  }
  // each lane keeps the scores of experts lane, lane+32, ... (E <= 1024 -> 32 per lane)
  float sc[MAX_EXPERTS / 32], sel[MAX_EXPERTS / 32];
#pragma unroll
  for (int j = 0; j < MAX_EXPERTS / 32; ++j) {
    const int e = j * 32 + lane;
    if (e < E) {
      sc[j] = fn == 0 ? __expf(row[e] - mx) / den : score_fn(row[e], fn);
      sel[j] = sc[j] + (bias ? bias[e] : 0.f);
    } else {
      sc[j] = 0.f;
      sel[j] = -INFINITY;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;
  int my_i = 0;
  for (int k = 0; k < K; ++k) {
    float best = -INFINITY;
    int be = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < MAX_EXPERTS / 32; ++j) {
      const int e = j * 32 + lane;
      if (sel[j] > best || (sel[j] == best && e < be)) { best = sel[j]; be = e; }
    }
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, be, o);
      if (ob > best || (ob == best && oe < be)) { best = ob; be = oe; }
    }
    // the owning lane reports the unbiased score and retires the expert
    float w = 0.f;
#pragma unroll
    for (int j = 0; j < MAX_EXPERTS / 32; ++j)
      if (j * 32 + lane == be) { w = sc[j]; sel[j] = -INFINITY; }
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    wsum += w;
    if (lane == k) { my_w = w; my_i = be; }
  }
  if (lane < K) {
    float w = my_w;
    if (fn != 0 && norm_topk) w /= wsum;
    idx[(size_t)t * K + lane] = my_i;
    wts[(size_t)t * K + lane] = w * route_scale;
  }
}

// Single block.  idx [R] global expert ids (R = T*K); experts [lo, hi) are local.
// Outputs: offsets [EL+1], route_row [R] (row in sorted order or -1), row_token [rows] (source token of a sorted row),
// work tables for token tiles of bn13 / bn2 rows, counts.
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ idx, int R, int K, int lo, int hi, int* __restrict__ offsets,
                int* __restrict__ route_row, int* __restrict__ row_token, int4* __restrict__ work13, int* __restrict__ n13,
                int m_tiles13, int bn13, int4* __restrict__ work2, int* __restrict__ n2, int m_tiles2, int bn2,
                int max_work) {
  __shared__ int cnt[MAX_EXPERTS], off[MAX_EXPERTS + 1], cur[MAX_EXPERTS], wbase13[MAX_EXPERTS + 1], wbase2[MAX_EXPERTS + 1];
  const int EL = hi - lo;
  for (int e = threadIdx.x; e < EL; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int r = threadIdx.x; r < R; r += blockDim.x) {
    const int e = idx[r] - lo;
    if (e >= 0 && e < EL) atomicAdd(&cnt[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int a = 0, w13 = 0, w2 = 0;
    for (int e = 0; e < EL; ++e) {
      off[e] = a;
      wbase13[e] = w13;
      wbase2[e] = w2;
      a += cnt[e];
      w13 += m_tiles13 * ((cnt[e] + bn13 - 1) / bn13);
      w2 += m_tiles2 * ((cnt[e] + bn2 - 1) / bn2);
    }
    off[EL] = a;
    wbase13[EL] = w13;
    wbase2[EL] = w2;
    *n13 = min(w13, max_work);
    *n2 = min(w2, max_work);
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= EL; e += blockDim.x) {
    offsets[e] = off[e];
    if (e < EL) cur[e] = 0;
  }
  __syncthreads();
  // stable placement: routes are scanned in order by one thread per expert to keep results run-to-run identical
  for (int e = threadIdx.x; e < EL; e += blockDim.x) {
    if (cnt[e] == 0) continue;
    int c = 0;
    for (int r = 0; r < R; ++r)
      if (idx[r] - lo == e) {
        route_row[r] = off[e] + c;
        row_token[off[e] + c] = r / K;
        ++c;
      }
  }
  for (int r = threadIdx.x; r < R; r += blockDim.x) {
    const int e = idx[r] - lo;
    if (e < 0 || e >= EL) route_row[r] = -1;
  }
  // work tables: m-tile fastest inside a token tile so one expert's weight tiles are swept once per token tile
  for (int e = threadIdx.x; e < EL; e += blockDim.x) {
    const int c = cnt[e];
    int w = wbase13[e];
    for (int nt = 0; nt * bn13 < c; ++nt)
      for (int m = 0; m < m_tiles13; ++m, ++w)
        if (w < max_work) work13[w] = make_int4(e, m, off[e] + nt * bn13, min(bn13, c - nt * bn13));
    w = wbase2[e];
    for (int nt = 0; nt * bn2 < c; ++nt)
      for (int m = 0; m < m_tiles2; ++m, ++w)
        if (w < max_work) work2[w] = make_int4(e, m, off[e] + nt * bn2, min(bn2, c - nt * bn2));
  }
}

// xs[row, :] = x[row_token[row], :]; one block per sorted row; H % 8 == 0.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_token,
                                  const int* __restrict__ offsets, int EL, __nv_bfloat16* __restrict__ xs, int H) {
  const int row = blockIdx.x;
  if (row >= offsets[EL]) return;
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row_token[row] * H);
  uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)row * H);
  for (int i = threadIdx.x; i < H / 8; i += blockDim.x) dst[i] = src[i];
}

__global__ void moe_swiglu_kernel(const __nv_bfloat16* __restrict__ gu, const int* __restrict__ offsets, int EL,
                                  __nv_bfloat16* __restrict__ act, int I, float limit) {
  const int row = blockIdx.x;
  if (row >= offsets[EL]) return;
  const __nv_bfloat16* g = gu + (size_t)row * 2 * I;
  const __nv_bfloat16* u = g + I;
  for (int i = threadIdx.x; i < I; i += blockDim.x) {
    float gv = __bfloat162float(g[i]), uv = __bfloat162float(u[i]);
    if (limit > 0.f) {
      uv = fminf(fmaxf(uv, -limit), limit);
      gv = fminf(gv, limit);
    }
    act[(size_t)row * I + i] = __float2bfloat16(gv / (1.f + __expf(-gv)) * uv);
  }
}

// out[t, :] = base[t, :] (optional) + sum_k wts[t,k] * y[route_row[t,k], :]
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_row,
                                   const float* __restrict__ wts, const __nv_bfloat16* __restrict__ base,
                                   __nv_bfloat16* __restrict__ out, int K, int H) {
  const int t = blockIdx.x;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    float acc = base ? __bfloat162float(base[(size_t)t * H + h]) : 0.f;
    for (int k = 0; k < K; ++k) {
      const int r = route_row[(size_t)t * K + k];
      if (r >= 0) acc += wts[(size_t)t * K + k] * __bfloat162float(y[(size_t)r * H + h]);
    }
    out[(size_t)t * H + h] = __float2bfloat16(acc);
  }
}

}  // namespace

extern "C" {

// score_fn: 0 softmax, 1 sigmoid, 2 sqrt(softplus). idx int32 [T, K], wts fp32 [T, K].
int b200_moe_route(const float* logits, const float* bias, int T, int E, int K, int score_fn, int norm_topk,
                   float route_scale, int* idx, float* wts, cudaStream_t stream) {
  if (T <= 0 || E <= 0 || E > MAX_EXPERTS || K <= 0 || K > MAX_TOPK || K > 32 || K > E) return -6;
  const int wpb = 4;
  moe_route_kernel<<<(T + wpb - 1) / wpb, wpb * 32, 0, stream>>>(logits, bias, T, E, K, score_fn, norm_topk, route_scale,
                                                               idx, wts);
  return (int)cudaGetLastError();
}

// Plans the grouped GEMMs of this rank's experts [expert_lo, expert_hi).  All outputs are device buffers:
// offsets int32 [EL+1]; route_row int32 [T*K]; row_token int32 [T*K]; work13 / work2: int4 [max_work]; n13 / n2: int32 [1].
int b200_moe_plan(const int* idx, int T, int K, int expert_lo, int expert_hi, int* offsets, int* route_row,
                  int* row_token, void* work13, int* n13, int m_tiles13, int bn13, void* work2, int* n2, int m_tiles2,
                  int bn2, int max_work, cudaStream_t stream) {
  const int EL = expert_hi - expert_lo;
  if (T <= 0 || K <= 0 || EL <= 0 || EL > MAX_EXPERTS || max_work <= 0) return -6;
  moe_plan_kernel<<<1, 1024, 0, stream>>>(idx, T * K, K, expert_lo, expert_hi, offsets, route_row, row_token,
                                          reinterpret_cast<int4*>(work13), n13, m_tiles13, bn13,
                                          reinterpret_cast<int4*>(work2), n2, m_tiles2, bn2, max_work);
  return (int)cudaGetLastError();
}

int b200_moe_gather(const void* x, const int* row_token, const int* offsets, int EL, void* xs, int max_rows, int H,
                    cudaStream_t stream) {
  if (max_rows <= 0 || H % 8) return -6;
  moe_gather_kernel<<<max_rows, 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(x), row_token, offsets, EL,
                                                  reinterpret_cast<__nv_bfloat16*>(xs), H);
  return (int)cudaGetLastError();
}

int b200_moe_swiglu(const void* gu, const int* offsets, int EL, void* act, int max_rows, int I, float limit,
                    cudaStream_t stream) {
  if (max_rows <= 0 || I <= 0) return -6;
  moe_swiglu_kernel<<<max_rows, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(gu), offsets, EL,
                                                  reinterpret_cast<__nv_bfloat16*>(act), I, limit);
  return (int)cudaGetLastError();
}

int b200_moe_combine(const void* y, const int* route_row, const float* wts, const void* base, void* out, int T, int K,
                     int H, cudaStream_t stream) {
  if (T <= 0 || K <= 0 || H <= 0) return -6;
  moe_combine_kernel<<<T, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(y), route_row, wts,
                                            reinterpret_cast<const __nv_bfloat16*>(base),
                                            reinterpret_cast<__nv_bfloat16*>(out), K, H);
  return (int)cudaGetLastError();
}

}  // extern "C"
