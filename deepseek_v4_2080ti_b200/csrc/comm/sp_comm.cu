// Sequence-parallel residual stream over peer memory: the owner-side half of the reduce-scatter and the
// all-gather that feeds the next column-parallel GEMM.
//
// Under tensor parallelism the reference keeps the hidden state replicated: every row-parallel projection ends in an
// all-reduce of the whole [T, H] tensor and every rank then runs the residual add and the RMSNorm on all T rows
// (cpp_engine/engine/qwen_engine.cpp:1942-2037 row-parallel + all-reduce, :3236-3245 replicated norms,
// src/models/deepseek_v4/runtime.py:824-878).  Here rank r owns rows [r*rows, (r+1)*rows) of the residual stream:
//   1. the row-parallel GEMM (gemm_wdec_kernel.cuh, ar_mode 3) pushes each partial tile to the owner of its rows;
//   2. sp_reduce_norm_gather_kernel (this file) waits for the tiles of its 8 rows, sums the partials in rank order,
//      adds them to the residual shard, normalises, and stores the normalised rows into the gathered activation
//      buffer of EVERY rank (plain 16-byte peer stores), then raises one flag per 8-row block on every peer;
//   3. the next column-parallel GEMM (ag_wait) reads its local gathered buffer, waiting for a block's flag first.
// Per sublayer a rank sends (W-1)/W of the [T, H] tensor twice (partials out, normalised rows out) - the volume of
// a bandwidth-optimal all-reduce - but the residual add and the norm run on T/W rows, and both transfers are
// issued from inside the producing kernels instead of a separate library collective.
// Every wait is bounded and reports ERR_WAIT_PEER through the status word; a kernel that finds the status word
// already set does not wait again.
#include <cuda_bf16.h>

#include "../ptx/sm100.cuh"
#include "comm.h"
#include "comm_device.cuh"
#include "sp_comm.h"

using namespace b200;

namespace {

constexpr int kRowsPerCta = B200_SP_FLAG_ROWS;   // one warp per row
constexpr int kThreads = kRowsPerCta * 32;

__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float2 v = __bfloat1622float2(h[k]);
    f[2 * k] = v.x;
    f[2 * k + 1] = v.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(f[2 * k], f[2 * k + 1]);
  return u;
}

// grid = rows / 8, block = 256.  h: this rank's residual shard [rows, H] (updated in place when partials are summed).
// with_partials: the kernel before this one on every rank was the reduce-scatter GEMM with token tile rs_bn and
// rs_m_tiles feature tiles; its epoch is the current ctrl[0].  The gathered rows go to result buffer `x_index` of
// every rank at row offset rank*rows.  gather == 0 keeps everything local (no peer store, no flag): used to fold the
// last partial sum into the residual.
__global__ void __launch_bounds__(kThreads)
sp_reduce_norm_gather_kernel(B200Comm c, __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ gamma,
                             float eps, int unit_offset, int rows, int H, int with_partials, int rs_bn, int rs_m_tiles,
                             int x_index, int gather, int epoch_word, int* status, uint64_t budget_ns) {
  const uint32_t prev = c.ctrl[0];
  const uint32_t epoch = prev + 1;
  // deferred gather: the push kernel, on another stream, raises the flags with this call's epoch
  if (epoch_word >= 0 && blockIdx.x == 0 && threadIdx.x == 0) c.ctrl[8 + epoch_word] = epoch;
  const int parity_p = prev & 1, parity_x = epoch & 1;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row0 = blockIdx.x * kRowsPerCta;
  __shared__ int failed;
  if (tid == 0) failed = 0;
  __syncthreads();
  if (with_partials) {
    const uint64_t budget = *reinterpret_cast<volatile int*>(status) == 0 ? budget_ns : 1000;
    const int nt = row0 / rs_bn;
    for (int i = tid; i < c.world * rs_m_tiles; i += kThreads) {
      const int src = i / rs_m_tiles, mt = i - src * rs_m_tiles;
      if (!wait_flag_ge(flag_slot(c.flags[c.rank], parity_p, src) + nt * rs_m_tiles + mt, prev, budget)) {
        atomicExch(status, ERR_WAIT_PEER);
        failed = 1;
      }
    }
    __syncthreads();
  }
  const int row = row0 + warp;
  if (!failed && row < rows) {
    const int nvec = H >> 3;
    __nv_bfloat16* hrow = h + (size_t)row * H;
    float ss = 0.f;
    if (with_partials) {
      const __nv_bfloat16* part0 = data_slot(c.data[c.rank], parity_p, 0, c.slot_elems) + (size_t)row * H;
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int r = 0; r < c.world; ++r) {
          float f[8];
          unpack8(__ldcg(reinterpret_cast<const uint4*>(part0 + (size_t)r * c.slot_elems + v * 8)), f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
        // same roundings as all-reduce followed by the fused add + norm: the reduced projection is a bf16 tensor,
        // and so is the residual stream
        float d[8], x[8];
        unpack8(pack8(acc), d);
        unpack8(*reinterpret_cast<const uint4*>(hrow + v * 8), x);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] += d[j];
        const uint4 o = pack8(x);
        *reinterpret_cast<uint4*>(hrow + v * 8) = o;
        unpack8(o, x);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
      }
    } else {
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        float x[8];
        unpack8(*reinterpret_cast<const uint4*>(hrow + v * 8), x);
#pragma unroll
        for (int j = 0; j < 8; ++j) ss += x[j] * x[j];
      }
    }
    if (gamma) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float inv = rsqrtf(ss / (float)H + eps);
      const size_t xoff = (size_t)x_index * c.slot_elems + ((size_t)c.rank * rows + row) * H;
#pragma unroll 2
      for (int v = lane; v < nvec; v += 32) {
        float x[8], g[8];
        unpack8(*reinterpret_cast<const uint4*>(hrow + v * 8), x);     // own stores of the first pass
        unpack8(__ldg(reinterpret_cast<const uint4*>(gamma + v * 8)), g);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = x[j] * inv * (unit_offset ? 1.f + g[j] : g[j]);
        const uint4 o = pack8(x);
        if (gather) {
          // peers first, starting with the next rank, so that the ranks' stores fan out over different links
          for (int k = 1; k <= c.world; ++k) {
            const int r = (c.rank + k) % c.world;
            *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(c.result[r]) + xoff + v * 8) = o;
          }
        } else {
          *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(c.result[c.rank]) + xoff + v * 8) = o;
        }
      }
      if (gather) __threadfence_system();
    }
  }
  __syncthreads();
  if (gather && gamma && !failed && tid < c.world && tid != c.rank)
    st_release_sys(flag_slot(c.flags2[tid], parity_x, c.rank) + blockIdx.x, epoch);
  finish_epoch(c.ctrl, epoch);
}

// The all-gather push on its own: copies this rank's normalised rows (already in its own gathered buffer, written by
// the kernel above with gather == 0) into every peer's gathered buffer and raises the per-8-row flags there, with the
// epoch that call left in ctrl[8 + epoch_word].  Launched on a second stream, it overlaps the column-parallel GEMM
// that has already started on this rank's own rows: that GEMM waits for the peers' flags tile by tile.
// grid-stride over 8-row blocks; 16-byte loads of a block, W-1 stores each, one system-scope release per block.
__global__ void __launch_bounds__(256)
sp_push_rows_kernel(B200Comm c, int rows, int H, int x_index, int epoch_word) {
  const uint32_t epoch = c.ctrl[8 + epoch_word];
  const int parity_x = epoch & 1;
  const int nvec = (kRowsPerCta * H) >> 3;            // 16-byte vectors per block (rows are contiguous)
  const size_t base = (size_t)x_index * c.slot_elems + (size_t)c.rank * rows * H;
  const __nv_bfloat16* src0 = reinterpret_cast<const __nv_bfloat16*>(c.result[c.rank]) + base;
  for (int b = blockIdx.x; b < rows / kRowsPerCta; b += gridDim.x) {
    const size_t off = (size_t)b * kRowsPerCta * H;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 q = *reinterpret_cast<const uint4*>(src0 + off + (size_t)v * 8);
      for (int k = 1; k < c.world; ++k) {
        const int r = (c.rank + k) % c.world;
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(c.result[r]) + base + off + (size_t)v * 8) = q;
      }
    }
    __syncthreads();
    if (threadIdx.x > 0 && threadIdx.x < c.world) {
      __threadfence_block();
      const int r = (c.rank + threadIdx.x) % c.world;
      st_release_sys(flag_slot(c.flags2[r], parity_x, c.rank) + b, epoch);
    }
    __syncthreads();
  }
}

// One CTA: waits until every peer has raised the flags of its `nblocks` row blocks for the gather that ran last
// (epoch = current ctrl[0]).  After it, any kernel on this stream may read the whole gathered buffer.
__global__ void __launch_bounds__(256)
sp_wait_gather_kernel(B200Comm c, int nblocks, int* status, uint64_t budget_ns) {
  const uint32_t epoch = c.ctrl[0];
  const int parity = epoch & 1;
  const uint64_t budget = *reinterpret_cast<volatile int*>(status) == 0 ? budget_ns : 1000;
  for (int i = threadIdx.x; i < c.world * nblocks; i += blockDim.x) {
    const int src = i / nblocks, b = i - src * nblocks;
    if (src == c.rank) continue;
    if (!wait_flag_ge(flag_slot(c.flags2[c.rank], parity, src) + b, epoch, budget)) atomicExch(status, ERR_WAIT_PEER);
  }
}

}  // namespace

extern "C" {

int b200_sp_push_rows(const B200Comm* c, int rows, int H, int x_index, int epoch_word, cudaStream_t stream) {
  if (!c || rows <= 0 || rows % kRowsPerCta || H % 8 || x_index < 0 || x_index > 1 || epoch_word < 0 || epoch_word > 3)
    return -ERR_BAD_ARG;
  if (c->world <= 1) return 0;
  int blocks = rows / kRowsPerCta;
  if (blocks > 64) blocks = 64;       // a quarter of the SMs' thread slots: the GEMM running beside it keeps the rest
  sp_push_rows_kernel<<<blocks, 256, 0, stream>>>(*c, rows, H, x_index, epoch_word);
  return (int)cudaGetLastError();
}

int b200_sp_reduce_norm_gather(const B200Comm* c, void* h_shard, const void* gamma, float eps, int unit_offset,
                               int rows, int H, int with_partials, int rs_bn, int x_index, int gather, int epoch_word,
                               int* status, unsigned long long budget_ns, cudaStream_t stream) {
  if (!c || rows <= 0 || rows % kRowsPerCta || H % 8 || x_index < 0 || x_index > 1 || !h_shard) return -ERR_BAD_ARG;
  if (epoch_word > 3) return -ERR_BAD_ARG;
  if ((unsigned long long)rows * c->world * H > c->slot_elems) return -ERR_BAD_ARG;
  if (rows / kRowsPerCta > B200_FLAGS_PER_SLOT) return -ERR_BAD_ARG;
  const int m_tiles = (H + 127) / 128;
  if (with_partials && (rs_bn <= 0 || rows % rs_bn || (long long)(rows / rs_bn) * m_tiles > B200_FLAGS_PER_SLOT))
    return -ERR_BAD_ARG;
  if (budget_ns == 0) budget_ns = B200_WAIT_BUDGET_NS;
  sp_reduce_norm_gather_kernel<<<rows / kRowsPerCta, kThreads, 0, stream>>>(
      *c, reinterpret_cast<__nv_bfloat16*>(h_shard), reinterpret_cast<const __nv_bfloat16*>(gamma), eps, unit_offset,
      rows, H, with_partials, rs_bn, m_tiles, x_index, gather, epoch_word, status, budget_ns);
  return (int)cudaGetLastError();
}

int b200_sp_wait_gather(const B200Comm* c, int rows, int* status, unsigned long long budget_ns, cudaStream_t stream) {
  if (!c || rows <= 0 || rows % kRowsPerCta) return -ERR_BAD_ARG;
  if (c->world == 1) return 0;
  if (budget_ns == 0) budget_ns = B200_WAIT_BUDGET_NS;
  sp_wait_gather_kernel<<<1, 256, 0, stream>>>(*c, rows / kRowsPerCta, status, budget_ns);
  return (int)cudaGetLastError();
}

}  // extern "C"
