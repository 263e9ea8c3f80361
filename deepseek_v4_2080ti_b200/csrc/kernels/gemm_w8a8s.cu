// Weight-streaming FP8 GEMM for small token counts (decode and speculative-verify batches):
//   Y[T, N] = X[T, K] * W[N, K]^T,  W = FP8 E4M3 with one scale per 128x128 block,  T <= 32.
//
// In this regime the kernel is bound by how fast the weight bytes leave HBM, so nothing may
// touch them between the bulk copy and the tensor core:
//   * the 8 KB weight tiles ([128 features x 64 K-bytes], stored pre-swizzled, see gemm_wdec.cu)
//     are copied two at a time (one 128-wide K block, 16 KB contiguous) into a deep shared-memory
//     ring (up to 12 slots, > 190 KB in flight per SM) and consumed by tcgen05.mma kind::f8f6f4 as
//     they are;
//   * the activations are what gets adapted: each bf16 row is split into 2 or 3 E4M3 terms
//     (x*c ~= hi + mid/16 + lo/256 with a per-row scale c), every term is one column of the
//     MMA's N dimension, and the epilogue recombines the columns.  Three terms carry ~12 bits
//     of significand, two terms ~8 bits (what a bf16 activation has);
//   * the 128x128 block scales are applied outside the tensor core: every 128-wide K block is
//     accumulated into its own TMEM buffer (one per ring slot), and the epilogue warps add
//     `scale * partial` into fp32 registers while the MMA warp is already on the next blocks;
//   * synchronisation is per K block, not per 64-byte stage: tcgen05.commit costs a few hundred
//     cycles of tensor-pipe time each, so one commit per block both frees the ring slot for the
//     producer and tells the epilogue that the block's accumulator is ready.
// Roles: warps 0-3 epilogue, warp 4 copy producer, warp 5 MMA issuer.  All waits are bounded.
//
// Reference behaviour covered: the FP8 block-128 matvec / small-batch kernels of the Qwen path
// (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:130-535), which dequantise in CUDA cores.
#include <cuda_bf16.h>
#include "per_device.h"
#include <cuda_fp8.h>
#include "../ptx/sm100.cuh"
#include <string.h>
#include "tma_host.h"
#include "ops.h"
#include "launch.h"
#include "../comm/comm.h"
#include "../comm/comm_device.cuh"

namespace b200 {
namespace w8s {

constexpr int BM = 128;            // output features per tile
constexpr int BKB = 64;            // K bytes (= fp8 elements) per stage
constexpr int W_BYTES = BM * BKB;  // 8 KB
constexpr int THREADS = 192;

struct Params {
  int T, N, K;
  int m_tiles, splits, kblk_total;   // kblk = 128-wide K blocks
  const uint8_t* w_tiled;
  const float* scales;
  int scale_ld;
  const float* inv_c;                // [T] 1 / activation scale
  __nv_bfloat16* out;                // [T, N]
  float* partial;                    // [splits, T, N] (splits > 1)
  const __nv_bfloat16* residual;
  int* tile_counters;
  int* status;
  // Fused one-shot all-reduce (row-parallel projection of a decode step under tensor parallelism): the CTA that
  // holds a finished 128-feature tile stores it as bf16 into its own slot and every peer's slot for source = this
  // rank, raises the tile's flag on the peers, waits for theirs and writes sum over ranks (+ residual) to `out`.
  int ar;
  unsigned long long ar_budget_ns;
  B200Comm comm;
};

template <int BN>
struct Smem {
  static constexpr int X_BYTES = BN * BKB;             // one 64-byte-wide activation tile
  static constexpr int SLOT = 2 * (W_BYTES + X_BYTES); // one 128-wide K block
  static constexpr int BUDGET = 232448 - 1024 - 1024;
  static constexpr int S_SMEM = BUDGET / SLOT;
  static constexpr int S_TMEM = 512 / BN;              // every slot owns BN accumulator columns
  static constexpr int S_MIN = S_SMEM < S_TMEM ? S_SMEM : S_TMEM;
  static constexpr int S = S_MIN > 12 ? 12 : S_MIN;
  static constexpr int TOTAL = S * SLOT + 1024 + 1024;
};

// K-major operand with the 64-byte swizzle: rows of 64 bytes, 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t desc_sw64(const void* smem_tile) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(smem_tile) & 0x3FFFF) >> 4);
  d |= (uint64_t)(512 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)4 << 61;   // SWIZZLE_64B
  return d;
}

// AR: the epilogue carries the one-shot all-reduce (instantiated for the narrow decode tiles only, so that the plain
// instances keep the code they had without it).
template <int BN, int TERMS, bool AR = false>
__global__ void __launch_bounds__(THREADS, 1)
gemm_w8a8s_kernel(const __grid_constant__ CUtensorMap tmX, Params p) {
  using L = Smem<BN>;
  constexpr int S = L::S;
  constexpr uint32_t TMEM_COLS = S * BN <= 32 ? 32 : S * BN <= 64 ? 64 : S * BN <= 128 ? 128 : S * BN <= 256 ? 256 : 512;
  constexpr int TOK = BN / TERMS;   // token slots per tile
  extern __shared__ uint8_t smem_raw_base[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_base) + 1023) & ~uintptr_t(1023));
  uint8_t* sW = smem;
  uint8_t* sX = sW + S * 2 * W_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sX + S * 2 * L::X_BYTES);
  uint64_t* full = bars;             // [S] copies of the block landed
  uint64_t* done = bars + S;         // [S] MMAs of the block finished: slot reusable, accumulator readable
  uint64_t* acc_free = bars + 2 * S; // [S] epilogue has read the accumulator
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 3 * S);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* epi_abort = abort_flag + 1;     // written by epilogue threads only, always before a barrier
  int* fix_last = const_cast<int*>(abort_flag) + 2;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&done[s], 1);
      mbar_init(&acc_free[s], 128);
    }
    *abort_flag = 0;
    *epi_abort = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == 4 && lane == 0) tma_prefetch_desc(&tmX);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();   // the next kernel may be scheduled; it waits for this grid before touching memory

  const int total_work = p.m_tiles * p.splits;
  const int per_split = (p.kblk_total + p.splits - 1) / p.splits;

  if (warp == 4) {
    // ------------------------------------------------------------ copy producer
    if (lane == 0) {
      // The weights do not depend on the previous kernel of the stream, the activations do.  When launched
      // as a programmatic dependent the producer therefore fills the ring with weight tiles first (up to S
      // blocks, ~190 KB per SM), waits for the predecessor, and only then fetches the activation tiles.
      const int pre = [&] {
        int n = 0;
        for (int w = blockIdx.x; w < total_work && n < S; w += gridDim.x) {
          const int m_tile = w % p.m_tiles, split = w / p.m_tiles;
          const int c0 = split * per_split, c1 = min(p.kblk_total, c0 + per_split);
          for (int c = c0; c < c1 && n < S; ++c, ++n) {
            mbar_expect_tx(&full[n], 2 * (W_BYTES + L::X_BYTES));
            bulk_load(sW + n * 2 * W_BYTES, p.w_tiled + ((size_t)m_tile * p.kblk_total + c) * (2 * W_BYTES),
                      2 * W_BYTES, &full[n]);
          }
        }
        return n;
      }();
      pdl_wait();
      uint32_t blk = 0;
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
        const int m_tile = w % p.m_tiles;
        const int split = w / p.m_tiles;
        const int c0 = split * per_split;
        const int c1 = min(p.kblk_total, c0 + per_split);
        const uint8_t* wsrc = p.w_tiled + ((size_t)m_tile * p.kblk_total + c0) * (2 * W_BYTES);
        for (int c = c0; c < c1; ++c, ++blk, wsrc += 2 * W_BYTES) {
          const int b = blk % S;
          if ((int)blk >= pre) {
            if (!mbar_wait(&done[b], ((blk / S) & 1) ^ 1)) {
              atomicExch(p.status, ERR_WAIT_STAGE);
              *abort_flag = 1;
              break;
            }
            mbar_expect_tx(&full[b], 2 * (W_BYTES + L::X_BYTES));
            // the two 64-byte-wide weight tiles of a K block are adjacent in memory: one 16 KB copy
            bulk_load(sW + b * 2 * W_BYTES, wsrc, 2 * W_BYTES, &full[b]);
          }
          tma_load_2d(sX + (2 * b) * L::X_BYTES, &tmX, &full[b], c * 128, 0);
          tma_load_2d(sX + (2 * b + 1) * L::X_BYTES, &tmX, &full[b], c * 128 + 64, 0);
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_e4m3(BM, BN);
      uint32_t blk = 0;
      bool failed = false;
      for (int w = blockIdx.x; w < total_work && !failed && !*abort_flag; w += gridDim.x) {
        const int split = w / p.m_tiles;
        const int c0 = split * per_split;
        const int c1 = min(p.kblk_total, c0 + per_split);
        for (int c = c0; c < c1; ++c, ++blk) {
          const int b = blk % S;
          const uint32_t ph = (blk / S) & 1;
          if (!mbar_wait(&acc_free[b], ph ^ 1)) {
            atomicExch(p.status, ERR_WAIT_ACC);
            failed = true;
            break;
          }
          if (!mbar_wait(&full[b], ph)) {
            atomicExch(p.status, ERR_WAIT_TMA);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + b * BN;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint64_t da = desc_sw64(sW + (2 * b + h) * W_BYTES);
            const uint64_t db = desc_sw64(sX + (2 * b + h) * L::X_BYTES);
            // one instruction covers 32 K-bytes: +32 bytes = +2 in 16-byte units
            umma_f8_ss(tmem_d, da, db, idesc, h);
            umma_f8_ss(tmem_d, da + 2, db + 2, idesc, 1u);
          }
          umma_commit(&done[b]);
        }
      }
      if (failed) *abort_flag = 1;
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    const int row = warp * 32 + lane;
    const bool sync_mode = p.splits > 1 || AR;
    pdl_wait();   // everything this role reads (inv_c, residual) or writes belongs after the previous kernel
    const uint32_t ar_epoch = AR ? p.comm.ctrl[0] + 1 : 0;   // after the wait: the previous kernel may have advanced it
    const int ar_parity = ar_epoch & 1;
    uint32_t blk = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      if (sync_mode) {
        if (threadIdx.x == 0 && *abort_flag) *epi_abort = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*epi_abort) break;
      } else if (*abort_flag) {
        break;
      }
      const int m_tile = w % p.m_tiles;
      const int split = w / p.m_tiles;
      const int c0 = split * per_split;
      const int c1 = min(p.kblk_total, c0 + per_split);
      const float* srow = p.scales + (size_t)m_tile * p.scale_ld;
      float acc[BN];
#pragma unroll
      for (int j = 0; j < BN; ++j) acc[j] = 0.f;
      float sc_next = (c0 < c1) ? __ldg(srow + c0) : 0.f;
      float my_inv_c[TOK];   // fetched now so the latency is hidden behind the main loop
#pragma unroll
      for (int t = 0; t < TOK; ++t) my_inv_c[t] = (t < p.T) ? __ldg(p.inv_c + t) : 0.f;
      bool ok = true;
      for (int c = c0; c < c1; ++c, ++blk) {
        const float sc = sc_next;
        if (c + 1 < c1) sc_next = __ldg(srow + c + 1);
        const int b = blk % S;
        ok = mbar_wait(&done[b], (blk / S) & 1);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        const uint32_t taddr = tmem_base + (uint32_t(warp * 32) << 16) + b * BN;
        if constexpr (BN == 16) {
          uint32_t v[16];
          tmem_ld_32x16(taddr, v);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[j] = fmaf(sc, __uint_as_float(v[j]), acc[j]);
        } else {
#pragma unroll
          for (int q = 0; q < BN / 32; ++q) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + q * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[q * 32 + j] = fmaf(sc, __uint_as_float(v[j]), acc[q * 32 + j]);
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_free[b]);
      }
      if (!ok) {
        if (lane == 0) atomicExch(p.status, ERR_WAIT_ACC);
        *abort_flag = 1;
        if (!sync_mode) break;
        *epi_abort = 1;
      }
      if (sync_mode) {
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*epi_abort) break;
      }
      // recombine the activation terms: column t*TERMS + j carries term j of token t
      const int f = m_tile * BM + row;
      const bool f_ok = f < p.N;
#pragma unroll
      for (int t = 0; t < TOK; ++t) {
        if (t < p.T && f_ok) {
          float v = acc[t * TERMS] + acc[t * TERMS + 1] * 0.0625f;
          if constexpr (TERMS == 3) v += acc[t * TERMS + 2] * 0.00390625f;
          v *= my_inv_c[t];
          const size_t off = (size_t)t * p.N + f;
          if (p.splits > 1) {
            p.partial[(size_t)split * p.T * p.N + off] = v;
          } else if (AR) {
            const __nv_bfloat16 bv = __float2bfloat16(v);
            for (int r = 0; r < p.comm.world; ++r) data_slot(p.comm.data[r], ar_parity, p.comm.rank, p.comm.slot_elems)[off] = bv;
          } else {
            if (p.residual) v += __bfloat162float(p.residual[off]);
            p.out[off] = __float2bfloat16(v);
          }
        }
      }
      bool tile_final = p.splits == 1;
      if (p.splits > 1) {
        // split-K fix-up by the CTA that arrives last at this tile (sums in split order: deterministic)
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (threadIdx.x == 0) {
          const int prev = atomicAdd(&p.tile_counters[m_tile], 1);
          *fix_last = (prev == p.splits - 1);
          if (prev == p.splits - 1) p.tile_counters[m_tile] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        tile_final = *fix_last != 0;
        if (*fix_last && f_ok) {
          __threadfence();
          for (int t = 0; t < p.T; ++t) {
            const size_t off = (size_t)t * p.N + f;
            float a = (p.residual && !AR) ? __bfloat162float(p.residual[off]) : 0.f;
            for (int sp = 0; sp < p.splits; ++sp) a += __ldcg(p.partial + (size_t)sp * p.T * p.N + off);
            if (AR) {
              const __nv_bfloat16 bv = __float2bfloat16(a);
              for (int r = 0; r < p.comm.world; ++r) data_slot(p.comm.data[r], ar_parity, p.comm.rank, p.comm.slot_elems)[off] = bv;
            } else {
              p.out[off] = __float2bfloat16(a);
            }
          }
        }
      }
      if (AR && tile_final) {
        // ---- the tile's all-reduce: flags out, flags in, sum in rank order (identical bits on every rank)
        const B200Comm& cm = p.comm;
        __threadfence_system();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int et = threadIdx.x;
        if (et < cm.world && et != cm.rank) {
          st_release_sys(flag_slot(cm.flags[et], ar_parity, cm.rank) + m_tile, ar_epoch);
          // once any kernel has recorded an expired wait the step is lost: do not spend the budget again
          const uint64_t budget = *reinterpret_cast<volatile int*>(p.status) == 0 ? p.ar_budget_ns : 1000;
          if (!wait_flag_ge(flag_slot(cm.flags[cm.rank], ar_parity, et) + m_tile, ar_epoch, budget)) {
            atomicExch(p.status, ERR_WAIT_PEER);
            *abort_flag = 1;
            *epi_abort = 1;
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*epi_abort) break;
        if (f_ok) {
          for (int t = 0; t < p.T; ++t) {
            const size_t off = (size_t)t * p.N + f;
            float a = p.residual ? __bfloat162float(p.residual[off]) : 0.f;
            for (int r = 0; r < cm.world; ++r)
              a += __bfloat162float(__ldcg(data_slot(cm.data[cm.rank], ar_parity, r, cm.slot_elems) + off));
            p.out[off] = __float2bfloat16(a);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // let copies that may still be in flight land before shared memory is released
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (AR && threadIdx.x == 0) {
    // the last CTA to leave publishes the new epoch (every epilogue read the old one before any CTA could leave)
    __threadfence();
    const uint32_t old = p.comm.ctrl[0];
    const uint32_t left = atomicAdd(&p.comm.ctrl[1], 1u) + 1;
    if (left == gridDim.x) {
      p.comm.ctrl[1] = 0;
      __threadfence();
      atomicExch(&p.comm.ctrl[0], old + 1);
    }
  }
}

// One block per token row: per-row scale c = 224 / max|x|, then TERMS successive E4M3 roundings of the
// residual, each 16x finer.  Output row t*TERMS + j holds term j; inside every 4-byte group the bytes are
// stored as (x0, x2, x1, x3), the order the packed weights use, so products pair up unchanged.
template <int TERMS>
__global__ void __launch_bounds__(256)
act_split_e4m3_kernel(const __nv_bfloat16* __restrict__ x, int K, uint8_t* __restrict__ xq,
                      float* __restrict__ inv_c) {
  pdl_launch_dependents();   // the GEMM that follows may start streaming its weights now
  pdl_wait();
  const int t = blockIdx.x;
  const __nv_bfloat16* xr = x + (size_t)t * K;
  __shared__ float red[8];
  float m = 0.f;
  for (int i = threadIdx.x * 4; i < K; i += 256 * 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    m = fmaxf(m, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))));
  }
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, red[i]);
  const float c = m > 0.f ? 224.f / m : 1.f;
  if (threadIdx.x == 0) inv_c[t] = 1.f / c;
  for (int i = threadIdx.x * 4; i < K; i += 256 * 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(xr + i);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    float v[4] = {a.x * c, a.y * c, b.x * c, b.y * c};
#pragma unroll
    for (int j = 0; j < TERMS; ++j) {
      uint8_t q[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const __nv_fp8_e4m3 f8(v[e]);
        q[e] = f8.__x;
        v[e] = (v[e] - float(f8)) * 16.f;
      }
      const uint32_t packed = (uint32_t)q[0] | ((uint32_t)q[2] << 8) | ((uint32_t)q[1] << 16) | ((uint32_t)q[3] << 24);
      *reinterpret_cast<uint32_t*>(xq + ((size_t)t * TERMS + j) * K + i) = packed;
    }
  }
}

template <int BN, int TERMS, bool AR = false>
static int launch(const CUtensorMap& tmX, const Params& p, cudaStream_t stream) {
  using L = Smem<BN>;
  static b200::PerDeviceOnce once_;
  bool& configured = once_.slot();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_w8a8s_kernel<BN, TERMS, AR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int total = p.m_tiles * p.splits;
  const int grid = total < sm_count() ? total : sm_count();
  // programmatic dependent launch: start while the kernel that produces the activations is still running
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&cfg, gemm_w8a8s_kernel<BN, TERMS, AR>, tmX, p);
}

}  // namespace w8s
}  // namespace b200

using namespace b200;

// Column layout chosen for a token count: returns BN (0 when T is out of range) and the term count.
extern "C" int b200_gemm_w8a8s_layout(int T, int* terms) {
  int bn = 0, tm = 2;
  if (T <= 5) { bn = 16; tm = 3; }
  else if (T <= 8) { bn = 16; tm = 2; }
  else if (T <= 16) { bn = 32; tm = 2; }
  else if (T <= 32) { bn = 64; tm = 2; }
  if (terms) *terms = tm;
  return bn;
}

// Split every bf16 row of x [T, K] into E4M3 terms: xq [T*terms, K] bytes, inv_c [T] floats.
extern "C" int b200_act_split_e4m3(const void* x_bf16, int T, int K, int terms, void* xq, float* inv_c,
                                   cudaStream_t stream) {
  if (T <= 0 || K <= 0 || (K % 4) != 0 || (terms != 2 && terms != 3)) return -ERR_BAD_ARG;
  const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(x_bf16);
  if (terms == 3)
    return (int)launch_pdl(w8s::act_split_e4m3_kernel<3>, dim3(T), dim3(256), 0, stream, x, K, reinterpret_cast<uint8_t*>(xq), inv_c);
  return (int)launch_pdl(w8s::act_split_e4m3_kernel<2>, dim3(T), dim3(256), 0, stream, x, K, reinterpret_cast<uint8_t*>(xq), inv_c);
}

// Y = X W^T with pre-split activations (b200_act_split_e4m3 with the layout of b200_gemm_w8a8s_layout(T)).
// W: FP8 tile-major packed weights (layout of b200_gemm_wdec, wfmt 1), scales fp32 [ceil(N/128), K/128].
// splits > 1 needs `partial` (splits*T*N floats) and `tile_counters` (ceil(N/128) zeroed ints, left zeroed).
static int gemm_w8a8s_launch(const void* W, const float* scales, const void* xq, const float* inv_c,
                             void* out_bf16, const void* residual, int T, int N, int K, int splits,
                             float* partial, int* tile_counters, const B200Comm* comm, unsigned long long budget_ns,
                             int* status, cudaStream_t stream);

extern "C" int b200_gemm_w8a8s(const void* W, const float* scales, const void* xq, const float* inv_c,
                               void* out_bf16, const void* residual, int T, int N, int K, int splits,
                               float* partial, int* tile_counters, int* status, cudaStream_t stream) {
  return gemm_w8a8s_launch(W, scales, xq, inv_c, out_bf16, residual, T, N, K, splits, partial, tile_counters, nullptr, 0,
                           status, stream);
}

// Row-parallel form: every rank calls it with its K-shard; all ranks end with out = sum over ranks (+ residual), the
// one-shot all-reduce done tile by tile in the epilogue over peer memory.  T * N <= comm->slot_elems.
extern "C" int b200_gemm_w8a8s_allreduce(const void* W, const float* scales, const void* xq, const float* inv_c,
                                         void* out_bf16, const void* residual, int T, int N, int K, int splits,
                                         float* partial, int* tile_counters, const B200Comm* comm,
                                         unsigned long long budget_ns, int* status, cudaStream_t stream) {
  if (!comm || comm->world <= 1)
    return gemm_w8a8s_launch(W, scales, xq, inv_c, out_bf16, residual, T, N, K, splits, partial, tile_counters, nullptr,
                             0, status, stream);
  if ((unsigned long long)T * N > comm->slot_elems || (N + w8s::BM - 1) / w8s::BM > B200_FLAGS_PER_SLOT) return -ERR_BAD_ARG;
  return gemm_w8a8s_launch(W, scales, xq, inv_c, out_bf16, residual, T, N, K, splits, partial, tile_counters, comm,
                           budget_ns ? budget_ns : B200_WAIT_BUDGET_NS, status, stream);
}

static int gemm_w8a8s_launch(const void* W, const float* scales, const void* xq, const float* inv_c,
                             void* out_bf16, const void* residual, int T, int N, int K, int splits,
                             float* partial, int* tile_counters, const B200Comm* comm, unsigned long long budget_ns,
                             int* status, cudaStream_t stream) {
  int terms = 0;
  const int BN = b200_gemm_w8a8s_layout(T, &terms);
  if (T <= 0 || BN == 0 || N <= 0 || K <= 0 || (K % 128) != 0 || splits < 1 || !out_bf16) return -ERR_BAD_ARG;
  w8s::Params p;
  p.T = T; p.N = N; p.K = K;
  p.m_tiles = (N + w8s::BM - 1) / w8s::BM;
  p.kblk_total = K / 128;
  if (splits > p.kblk_total) splits = p.kblk_total;
  {
    const int per = (p.kblk_total + splits - 1) / splits;
    splits = (p.kblk_total + per - 1) / per;   // no empty split
  }
  p.splits = splits;
  if (splits > 1 && (!partial || !tile_counters)) return -ERR_BAD_ARG;
  p.w_tiled = reinterpret_cast<const uint8_t*>(W);
  p.scales = scales;
  p.scale_ld = K / 128;
  p.inv_c = inv_c;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.partial = partial;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.tile_counters = tile_counters;
  p.status = status;
  p.ar = comm ? 1 : 0;
  p.ar_budget_ns = budget_ns;
  memset(&p.comm, 0, sizeof(p.comm));
  if (comm) p.comm = *comm;
  CUtensorMap tmX;
  if (!make_tmap_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, xq, (uint64_t)T * terms, K, (uint64_t)K, BN, w8s::BKB,
                    CU_TENSOR_MAP_SWIZZLE_64B))
    return -ERR_BAD_ARG;
  if (p.ar) {
    if (BN != 16) return -ERR_BAD_ARG;       // the fused all-reduce exists for up to 8 tokens
    return terms == 3 ? w8s::launch<16, 3, true>(tmX, p, stream) : w8s::launch<16, 2, true>(tmX, p, stream);
  }
  if (BN == 16 && terms == 3) return w8s::launch<16, 3>(tmX, p, stream);
  if (BN == 16) return w8s::launch<16, 2>(tmX, p, stream);
  if (BN == 32) return w8s::launch<32, 2>(tmX, p, stream);
  return w8s::launch<64, 2>(tmX, p, stream);
}
