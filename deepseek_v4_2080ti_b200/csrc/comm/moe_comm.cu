// Expert-parallel combine fused with its collective, over peer memory.
//
// Experts are sharded by range over the ranks and every rank holds every token (the activations are replicated by the
// preceding attention all-reduce), so the "dispatch" half of expert parallelism is a local gather; what crosses
// NVLink is the combine: out[t] = residual[t] + sum over ranks of (shared-expert partial + sum_k w[t,k] * y_local[row]).
// One kernel computes each rank's weighted partial rows and moves them:
//   * one-shot (small T, decode): the partial of every row chunk is pushed into every peer's slot, each rank sums;
//   * two-shot (prefill): chunk c belongs to rank c % world; partials go only to the owner, which sums them and
//     pushes the finished rows to everyone (total traffic per rank 2 (W-1)/W of the payload instead of (W-1)).
// Nothing waits on a CTA of the same GPU, every CTA first pushes all of its chunks and only then waits, and all
// waits are bounded: a missing peer ends the kernel with ERR_WAIT_PEER in the status word.
// The reference's counterpart is "expert-range sharding + all-reduce" (src/models/deepseek_v4/runtime.py:3664-4274,
// src/models/minimax_m2/architecture.py:367-384) with the combine, the NCCL all-reduce and the residual add as
// separate kernels.
#include <cuda_bf16.h>

#include "comm_device.cuh"

using namespace b200;

namespace {

constexpr int kThreads = 256;

// Weighted partial of one row segment: 8 consecutive features of token t.
__device__ __forceinline__ void partial8(const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_row,
                                         const float* __restrict__ wts, const __nv_bfloat16* __restrict__ base, int t,
                                         int K, int H, int h, float acc[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) acc[j] = 0.f;
  if (base) {
    const uint4 u = *reinterpret_cast<const uint4*>(base + (size_t)t * H + h);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(p[j]);
      acc[2 * j] += f.x;
      acc[2 * j + 1] += f.y;
    }
  }
  for (int k = 0; k < K; ++k) {
    const int r = route_row[(size_t)t * K + k];
    if (r < 0) continue;
    const float w = wts[(size_t)t * K + k];
    const uint4 u = *reinterpret_cast<const uint4*>(y + (size_t)r * H + h);
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __bfloat1622float2(p[j]);
      acc[2 * j] += w * f.x;
      acc[2 * j + 1] += w * f.y;
    }
  }
}

__device__ __forceinline__ uint4 pack8(const float acc[8]) {
  uint4 u;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) p[j] = __floats2bfloat162_rn(acc[2 * j], acc[2 * j + 1]);
  return u;
}

__device__ __forceinline__ void add8(float acc[8], const uint4& u) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __bfloat1622float2(p[j]);
    acc[2 * j] += f.x;
    acc[2 * j + 1] += f.y;
  }
}

// chunk = `rows_per` consecutive token rows.  H % 8 == 0.
__global__ void __launch_bounds__(kThreads)
moe_combine_reduce_kernel(B200Comm c, const __nv_bfloat16* __restrict__ y, const int* __restrict__ route_row,
                          const float* __restrict__ wts, const __nv_bfloat16* __restrict__ base,
                          const __nv_bfloat16* __restrict__ residual, __nv_bfloat16* __restrict__ out, int T, int K, int H,
                          int rows_per, int chunks, int two_shot, int* status, uint64_t budget_ns) {
  const uint32_t epoch = c.ctrl[0] + 1;
  const int parity = epoch & 1;
  const int W = c.world, me = c.rank;
  const int vec_per_row = H / 8;
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();

  // ---- phase 1: partial rows of every chunk of this CTA -> the slot(s) that will sum them
  for (int ch = blockIdx.x; ch < chunks; ch += gridDim.x) {
    const int t0 = ch * rows_per, t1 = min(T, t0 + rows_per);
    const int owner = ch % W;
    for (int v = threadIdx.x; v < (t1 - t0) * vec_per_row; v += kThreads) {
      const int t = t0 + v / vec_per_row, h = (v % vec_per_row) * 8;
      float acc[8];
      partial8(y, route_row, wts, base, t, K, H, h, acc);
      const uint4 u = pack8(acc);
      const size_t off = (size_t)t * H + h;
      if (two_shot) {
        *reinterpret_cast<uint4*>(data_slot(c.data[owner], parity, me, c.slot_elems) + off) = u;
      } else {
        for (int r = 0; r < W; ++r) *reinterpret_cast<uint4*>(data_slot(c.data[r], parity, me, c.slot_elems) + off) = u;
      }
    }
    __threadfence_system();
    __syncthreads();
    if (two_shot) {
      if (threadIdx.x == 0 && owner != me) st_release_sys(flag_slot(c.flags[owner], parity, me) + ch, epoch);
    } else if (threadIdx.x < W && threadIdx.x != me) {
      st_release_sys(flag_slot(c.flags[threadIdx.x], parity, me) + ch, epoch);
    }
  }

  // ---- phase 2: sum the chunks this rank is responsible for (all of them in one-shot mode)
  for (int ch = blockIdx.x; ch < chunks; ch += gridDim.x) {
    const int owner = ch % W;
    if (two_shot && owner != me) continue;
    if (threadIdx.x < W && threadIdx.x != me) {
      if (!wait_flag_ge(flag_slot(c.flags[me], parity, threadIdx.x) + ch, epoch, budget_ns)) {
        atomicExch(status, ERR_WAIT_PEER);
        failed = 1;
      }
    }
    __syncthreads();
    if (failed) break;
    const int t0 = ch * rows_per, t1 = min(T, t0 + rows_per);
    for (int v = threadIdx.x; v < (t1 - t0) * vec_per_row; v += kThreads) {
      const int t = t0 + v / vec_per_row, h = (v % vec_per_row) * 8;
      const size_t off = (size_t)t * H + h;
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (residual) add8(acc, *reinterpret_cast<const uint4*>(residual + off));
      for (int r = 0; r < W; ++r)   // fixed order: every rank gets bit-identical sums
        add8(acc, *reinterpret_cast<const uint4*>(data_slot(c.data[me], parity, r, c.slot_elems) + off));
      const uint4 u = pack8(acc);
      *reinterpret_cast<uint4*>(out + off) = u;
      if (two_shot)
        for (int r = 0; r < W; ++r)
          if (r != me) *reinterpret_cast<uint4*>(result_half(c.result[r], parity, c.slot_elems) + off) = u;
    }
    if (two_shot) {
      __threadfence_system();
      __syncthreads();
      if (threadIdx.x < W && threadIdx.x != me)
        st_release_sys(flag_slot(c.flags2[threadIdx.x], parity, me) + ch, epoch);
    }
  }

  // ---- phase 3 (two-shot): collect the finished chunks of the other owners
  if (two_shot && !failed) {
    for (int ch = blockIdx.x; ch < chunks; ch += gridDim.x) {
      const int owner = ch % W;
      if (owner == me) continue;
      if (threadIdx.x == 0 && !wait_flag_ge(flag_slot(c.flags2[me], parity, owner) + ch, epoch, budget_ns)) {
        atomicExch(status, ERR_WAIT_PEER);
        failed = 1;
      }
      __syncthreads();
      if (failed) break;
      const int t0 = ch * rows_per, t1 = min(T, t0 + rows_per);
      const __nv_bfloat16* src = result_half(c.result[me], parity, c.slot_elems);
      for (int v = threadIdx.x; v < (t1 - t0) * vec_per_row; v += kThreads) {
        const size_t off = (size_t)(t0 + v / vec_per_row) * H + (v % vec_per_row) * 8;
        *reinterpret_cast<uint4*>(out + off) = *reinterpret_cast<const uint4*>(src + off);
      }
      __syncthreads();
    }
  }
  finish_epoch(c.ctrl, epoch);
}

}  // namespace

extern "C" {

// out[t, :] = residual[t, :] + sum over ranks of ( base_r[t, :] + sum_k wts[t, k] * y_r[route_row_r[t, k], :] ), bf16.
//   y          bf16 [rows, H]   this rank's expert outputs in expert-sorted order
//   route_row  int32 [T, K]     row of y for route (t, k), or -1 when that expert lives on another rank
//   wts        fp32 [T, K]      routing weights (identical on every rank)
//   base       bf16 [T, H] or null: a per-rank partial added before the exchange (e.g. a TP-sharded shared expert)
//   residual   bf16 [T, H] or null: added once, after the sum
// T * H <= slot_elems, H % 8 == 0.  mode: 0 = pick by size, 1 = one-shot, 2 = two-shot.
int b200_moe_combine_allreduce(const B200Comm* c, const void* y, const int* route_row, const float* wts, const void* base,
                               const void* residual, void* out, int T, int K, int H, int mode, int* status,
                               unsigned long long budget_ns, cudaStream_t stream) {
  if (T <= 0 || K <= 0 || H <= 0 || (H % 8) != 0 || (unsigned long long)T * H > c->slot_elems) return -ERR_BAD_ARG;
  if (budget_ns == 0) budget_ns = B200_WAIT_BUDGET_NS;
  int two_shot = mode == 2 || (mode == 0 && c->world > 2 && (long long)T * H >= (1 << 18));
  if (c->world == 1) two_shot = 0;
  // chunk rows: about 16 KB per chunk, at most FLAGS_PER_SLOT chunks
  int rows_per = (8192 + H - 1) / H;
  if (rows_per < 1) rows_per = 1;
  while ((T + rows_per - 1) / rows_per > B200_FLAGS_PER_SLOT) rows_per *= 2;
  const int chunks = (T + rows_per - 1) / rows_per;
  // every CTA must be resident at once (a CTA's peers wait on it): 2 CTAs of 256 threads per SM fit easily
  const int grid = chunks < 296 ? chunks : 296;
  moe_combine_reduce_kernel<<<grid, kThreads, 0, stream>>>(
      *c, reinterpret_cast<const __nv_bfloat16*>(y), route_row, wts, reinterpret_cast<const __nv_bfloat16*>(base),
      reinterpret_cast<const __nv_bfloat16*>(residual), reinterpret_cast<__nv_bfloat16*>(out), T, K, H, rows_per, chunks,
      two_shot, status, budget_ns);
  return (int)cudaGetLastError();
}

}  // extern "C"
