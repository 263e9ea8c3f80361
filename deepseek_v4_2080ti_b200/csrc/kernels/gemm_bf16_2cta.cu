// Prefill-size bf16 GEMM on CTA pairs:  Y[T, N] = X[T, K] * W[N, K]^T  with tcgen05.mma.cta_group::2.
//
// Why a second GEMM kernel: the one-CTA tile of gemm_wdec_kernel.cuh (128 features x 256 tokens) moves 48 KB
// through shared memory per 64-wide k-block, in by TMA and out to the tensor core, and that traffic - not the tensor
// pipe - bounds it at ~0.64 of the measured cuBLAS rate.  A pair of CTAs on two SMs computes a 256-feature x 256-token
// tile with ONE instruction stream: each CTA stages its 128 weight rows and only HALF of the token tile (128 rows), the
// tensor cores of both SMs read the two token halves from both shared memories, and each SM accumulates its own 128
// features x 256 tokens in its own TMEM.  Shared-memory fill per k-block and SM drops from 48 KB to 32 KB for the same
// math, and six pipeline stages fit instead of four.
//
// Operand roles: tokens are the MMA's M dimension here (128 token rows per CTA = its TMEM lanes) and features the N
// dimension (256 columns), the other way round from gemm_wdec_kernel.cuh, whose 128-feature M tile exists for decode
// batches.  An epilogue thread then owns one token row and 32 consecutive features per TMEM read - 64 contiguous
// bytes of the row-major output - so it stores with four 16-byte instructions where the feature-per-thread layout
// needs thirty-two 2-byte ones (that store count, ~20 us per tile, bounds the one-CTA kernel whenever K is short).
//
// Structure (both CTAs of a pair run the same code; cluster rank 0 is the leader):
//   warp 4   TMA producer: own token half (A) + own feature half (B) per stage (cp.async.bulk.tensor, destination =
//            own shared memory, no multicast); the transaction bytes of BOTH CTAs complete on the leader's `full` barrier;
//   warp 5   leader only: one thread issues the cta_group::2 MMAs and commits; commits are multicast to the `empty`
//            and `acc_full` barriers of both CTAs (tcgen05.commit ... multicast::cluster);
//   warps 0-3 epilogue of the CTA's own 128 token rows x 256 features: TMEM -> bf16 -> 16-byte global stores; then one
//            remote arrive per warp on the leader's `acc_empty` barrier.
// Epilogue targets: the local output, or (reduce-scatter mode) the slot of the rank that owns those token rows plus a
// per-tile flag - the same protocol as gemm_wdec_kernel.cuh ar_mode 3, consumed by comm/sp_comm.cu.  The producer can
// also wait for the all-gather flags of its token half before loading it (ag_wait).
// Every wait is bounded; on expiry the CTA records the error word and leaves through the common exit (cluster barrier,
// TMEM freed by both CTAs).
//
// Reference behaviour covered: the FP8 -> fp16 dequant + cublasGemmEx prefill path
// (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:1199-1349).
#include <cuda_bf16.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "../comm/comm.h"
#include "../comm/comm_device.cuh"
#include "../ptx/sm100.cuh"
#include "gemm_2cta.h"
#include "per_device.h"
#include "tma_host.h"

namespace b200 {
namespace g2 {

constexpr int BM = 128;            // token rows per CTA (256 per pair): the MMA's M / 2
constexpr int BNH = 128;           // feature rows of W staged per CTA (256 per pair): the MMA's N / 2
constexpr int BN = 256;            // features per pair tile = accumulator columns
constexpr int BK = 64;
constexpr int S = 6;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = BNH * BK * 2;
constexpr int STAGE_BYTES = 4 * 32 * 256;   // reduce-scatter epilogue: per warp 32 token rows x 128 features of bf16
constexpr int SMEM_TOTAL = 1024 + S * (A_BYTES + B_BYTES) + 1024 + STAGE_BYTES;
constexpr int THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_bar_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}
// TMA load whose completion bytes are counted on a barrier of the pair's leader (address already mapped there).
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t leader_bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(tmap), "r"(leader_bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  const uint32_t z = 0;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5, %5, %5, %5, %5}, p;\n\t}\n"
      :
      : "r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(z)
      : "memory");
}
// Completion of this thread's earlier MMAs arrives on the barrier at the same offset in every CTA of `mask`.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar, uint16_t mask) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                   smem_u32(bar)),
               "h"(mask)
               : "memory");
}

struct Params {
  int T, N, K, kb_total, m2_tiles, n_tiles, ldo;
  __nv_bfloat16* out;
  int* status;
  int mode;               // 0: store to out; 3: reduce-scatter push (see gemm_wdec_kernel.cuh ar_mode 3);
                          // 4: W rows interleaved [gate tile | up tile]: out[T, N/2] = silu(gate) * up
  int n_rot, sp_rows;
  int ag_wait, ag_flag_rows;
  unsigned long long budget_ns;
  int tma_push;           // mode 3: push the staged tile with bulk tensor stores through `OutMaps` (else plain stores)
  int slot_rows;          // rows of `ldo` elements per (parity, source) data slot
  B200Comm comm;
};

// One tensor map per owner rank over that rank's whole data region, seen as [16 slots x slot_rows, ldo] bf16 with a
// box of 32 rows x 64 features (one warp's share of half a staging patch).  Stores only: a load through these maps
// would be a TMA load from peer memory, which this kernel never issues.
struct OutMaps {
  CUtensorMap m[B200_MAX_RANKS];
};

__device__ __forceinline__ void bulk_wait_read_1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_4() { asm volatile("cp.async.bulk.wait_group 4;" ::: "memory"); }

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_bf16_2cta_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const __grid_constant__ OutMaps omaps, Params p) {
  extern __shared__ uint8_t smem_raw_base[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_base) + 1023) & ~uintptr_t(1023));
  uint8_t* sA = smem;
  uint8_t* sB = sA + S * A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sB + S * B_BYTES);
  uint64_t* full = bars;               // [S]  leader: both CTAs' stage bytes landed
  uint64_t* empty = bars + S;          // [S]  each CTA: the stage's MMAs are done
  uint64_t* acc_full = bars + 2 * S;   // [2]  each CTA: accumulator ready
  uint64_t* acc_empty = bars + 2 * S + 2;  // [2] leader: both epilogues have drained the accumulator (8 warp arrives)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // epilogue warps that have stored their part of a tile, one counter per tile_i & 3: the four warps run up to two
  // tiles apart (the accumulator is double-buffered), so a single counter would mix arrivals of different tiles
  int* epi_count = const_cast<int*>(abort_flag) + 1;   // [4]
  uint8_t* sStage = reinterpret_cast<uint8_t*>(bars) + 1024;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], 8);
    }
    *abort_flag = 0;
    for (int i = 0; i < 4; ++i) epi_count[i] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 5) {
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  if (warp == 4 && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // the peer's barriers exist before anything is signalled across the pair
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t ar_epoch = p.mode == 3 ? p.comm.ctrl[0] + 1 : 0;
  // once any kernel has recorded an expired wait the step is lost: later kernels give up quickly instead of spending
  // the full budget at every barrier
  const uint64_t wait_ns = *reinterpret_cast<volatile int*>(p.status) == 0 ? p.budget_ns : 2000000ull;

  const int total = p.m2_tiles * p.n_tiles;
  // Tile order: bands of up to 16 feature tiles; inside a band the feature tile moves fastest, then the token tile.
  // The ~74 pairs in flight then share 16 weight tiles and ~5 token tiles (tens of MB, inside the 126 MB L2), and a
  // band's weights are read from HBM once; with the feature tile fastest over the whole width, a wide N (gate_up:
  // 136 tiles) makes every token tile stream the whole weight matrix from HBM again.
  auto tile_of = [&](int w, int& m2, int& nt) {
    constexpr int GM = 16;
    const int per_band = GM * p.n_tiles;
    const int band = w / per_band;
    const int r = w - band * per_band;
    const int in_band = min(GM, p.m2_tiles - band * GM);
    m2 = band * GM + r % in_band;
    nt = r / in_band + p.n_rot;
    if (nt >= p.n_tiles) nt -= p.n_tiles;
  };

  if (warp == 4) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    const uint32_t ag_epoch = p.ag_wait ? p.comm.ctrl[0] : 0;
    const uint64_t ag_budget = wait_ns;
    uint32_t it = 0;
    for (int w = pair; w < total; w += npairs) {
      int stop = (lane == 0) ? *abort_flag : 0;
      stop = __shfl_sync(0xffffffffu, stop, 0);
      if (stop) break;
      int m2, nt;
      tile_of(w, m2, nt);
      const int tok0 = nt * 2 * BM + (int)rank * BM;     // this CTA's half of the pair's 256 token rows
      if (p.ag_wait) {
        const int src = tok0 / p.sp_rows;
        if (src != p.comm.rank) {
          const int first = (tok0 - src * p.sp_rows) / p.ag_flag_rows;
          const int cnt = BM / p.ag_flag_rows;
          const uint32_t* fl = flag_slot(p.comm.flags2[p.comm.rank], ag_epoch & 1, src) + first;
          bool ok = true;
          for (int i = lane; i < cnt; i += 32) ok = ok && wait_flag_ge(fl + i, ag_epoch, ag_budget);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) {
              atomicExch(p.status, ERR_WAIT_PEER);
              *abort_flag = 1;
            }
            break;
          }
        }
      }
      int failed = 0;
      if (lane == 0) {
        for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, wait_ns)) {
            atomicExch(p.status, ERR_WAIT_STAGE);
            *abort_flag = 1;
            failed = 1;
            break;
          }
          if (leader) mbar_expect_tx(&full[s], 2 * (A_BYTES + B_BYTES));
          const uint32_t lbar = map_to_cta(smem_u32(&full[s]), 0);
          tma_load_2d_pair(sA + s * A_BYTES, &tmX, lbar, kb * BK, tok0);
          tma_load_2d_pair(sB + s * B_BYTES, &tmW, lbar, kb * BK, m2 * BN + (int)rank * BNH);
        }
      }
      failed = __shfl_sync(0xffffffffu, failed, 0);
      if (failed) break;
    }
    // tail: every commit aimed at this CTA's `empty` barriers must have landed before the CTA may exit
    if (lane == 0 && !*abort_flag) {
      const uint32_t done = it;
      for (uint32_t j = (done > (uint32_t)S ? done - S : 0); j < done; ++j) mbar_wait(&empty[j % S], (j / S) & 1, wait_ns);
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer (leader CTA only)
    if (leader && lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(2 * BM, BN);
      uint32_t it = 0, tile_i = 0;
      for (int w = pair; w < total && !*abort_flag; w += npairs, ++tile_i) {
        const int buf = tile_i & 1;
        if (!mbar_wait(&acc_empty[buf], ((tile_i >> 1) & 1) ^ 1, wait_ns)) {
          atomicExch(p.status, ERR_WAIT_ACC);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        bool failed = false;
        for (int kb = 0; kb < p.kb_total; ++kb, ++it) {
          const int s = it % S;
          if (!mbar_wait(&full[s], (it / S) & 1, wait_ns)) {
            atomicExch(p.status, ERR_WAIT_TMA);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint64_t da = umma_desc_sw128(sA + s * A_BYTES);
          const uint64_t db = umma_desc_sw128(sB + s * B_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) umma_bf16_pair(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          umma_commit_pair(&empty[s], 3);
        }
        if (failed) {
          *abort_flag = 1;
          break;
        }
        umma_commit_pair(&acc_full[buf], 3);
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (both CTAs, own 128 token rows)
    const int row_in_tile = warp * 32 + lane;             // TMEM lane == token row within the CTA's half
    const uint32_t lead_acc_empty0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
    uint32_t tile_i = 0;
    // The last of the four warps to finish a tile raises its flags on the owner (no CTA-wide barrier: a warp that has
    // to give up does not strand the others).  Ordering: a warp's stores (complete, for bulk stores) -> __syncwarp ->
    // its lane 0 fences at CTA scope and counts itself in; the lane that counts fourth fences again and issues ONE
    // system-scope release, which by cumulativity covers the stores of all four warps.  (A system-scope fence per
    // thread per tile, the obvious form, measured ~15 us per tile at 2 ranks: 0.33 ms instead of 0.20 ms for
    // 8192 x 5120 x 2048.)  One counter per tile & 3: the warps run up to two tiles apart, and a deferred signal
    // trails by one more.
    auto signal_tile = [&](uint32_t t_i, int owner, int dst_row0, int m2) {
      __syncwarp();
      if (lane == 0) {
        __threadfence_block();
        if ((atomicAdd(&epi_count[t_i & 3], 1) & 3) == 3) {   // the counters only grow: four arrivals per tile
          __threadfence_block();
          // this CTA's 128 rows x 256 features = two 128-feature tiles of the 128-row block, as the owner counts them
          uint32_t* fl = flag_slot(p.comm.flags[owner], ar_epoch & 1, p.comm.rank) +
                         (dst_row0 / BM) * (p.m2_tiles * 2) + m2 * 2;
          st_release_sys(fl, ar_epoch);
          st_release_sys(fl + 1, ar_epoch);
        }
      }
    };
    bool have_prev = false;
    int prev_owner = 0, prev_row0 = 0, prev_m2 = 0;
    for (int w = pair; w < total && !*abort_flag; w += npairs, ++tile_i) {
      int m2, nt;
      tile_of(w, m2, nt);
      const int buf = tile_i & 1;
      bool ok = mbar_wait(&acc_full[buf], (tile_i >> 1) & 1, wait_ns);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) atomicExch(p.status, ERR_WAIT_ACC);
        *abort_flag = 1;
        break;
      }
      tc_fence_after();
      const int row0 = nt * 2 * BM + (int)rank * BM;      // first token row of this CTA's half
      __nv_bfloat16* dst;
      int dst_row0 = row0, owner = 0;
      if (p.mode == 3) {
        owner = row0 / p.sp_rows;
        dst_row0 = row0 - owner * p.sp_rows;
        dst = data_slot(p.comm.data[owner], ar_epoch & 1, p.comm.rank, p.comm.slot_elems);
      } else {
        dst = p.out;
      }
      __nv_bfloat16* drow = dst + (size_t)(dst_row0 + row_in_tile) * p.ldo + (size_t)m2 * BN;
      const uint32_t taddr = tmem_base + (uint32_t(warp * 32) << 16) + buf * BN;
      if (p.mode == 4) {
        // SwiGLU: accumulator columns [0, 128) are the gate and [128, 256) the up projection of the same 128
        // features; the activation is taken on the fp32 accumulators and only the product is written
        __nv_bfloat16* orow = p.out + (size_t)(row0 + row_in_tile) * p.ldo + (size_t)m2 * (BN / 2);
#pragma unroll 1
        for (int c0 = 0; c0 < BN / 2; c0 += 32) {
          uint32_t v[2][32];
          tmem_ld_32x32(taddr + c0, v[0]);
          tmem_ld_32x32(taddr + BN / 2 + c0, v[1]);
          tmem_ld_wait();
          if (c0 + 32 >= BN / 2) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) remote_arrive(lead_acc_empty0 + buf * 8);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float g0 = __uint_as_float(v[0][q4 * 8 + 2 * e]), g1 = __uint_as_float(v[0][q4 * 8 + 2 * e + 1]);
              const float u0 = __uint_as_float(v[1][q4 * 8 + 2 * e]), u1 = __uint_as_float(v[1][q4 * 8 + 2 * e + 1]);
              oh[e] = __floats2bfloat162_rn(g0 / (1.f + __expf(-g0)) * u0, g1 / (1.f + __expf(-g1)) * u1);
            }
            *reinterpret_cast<uint4*>(orow + c0 + q4 * 8) = o;
          }
        }
      } else if (p.mode != 3) {
        // two TMEM reads in flight per wait: the read latency, not the store count, paces this loop
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 64) {
          uint32_t v[2][32];
          tmem_ld_32x32(taddr + c0, v[0]);
          tmem_ld_32x32(taddr + c0 + 32, v[1]);
          tmem_ld_wait();
          if (c0 + 64 >= BN) {
            // accumulator drained: one arrive per warp on the leader's barrier
            tc_fence_before();
            __syncwarp();
            if (lane == 0) remote_arrive(lead_acc_empty0 + buf * 8);
          }
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                oh[e] = __floats2bfloat162_rn(__uint_as_float(v[hh][q4 * 8 + 2 * e]), __uint_as_float(v[hh][q4 * 8 + 2 * e + 1]));
              *reinterpret_cast<uint4*>(drow + c0 + hh * 32 + q4 * 8) = o;
            }
          }
        }
      } else if (p.tma_push) {
        // Bulk tensor stores: each warp turns 32 rows x 64 features into bf16 in one of its two 4 KB staging boxes
        // (128-byte rows, 16-byte chunks XOR-ed with row & 7 = the layout SWIZZLE_128B expects), and lane 0 hands the
        // box to the copy engine, which writes it into the owner's slot - 4 KB per instruction instead of 16 bytes
        // per thread, and the warp is free for the next 64 features while the bytes cross NVLink.  A box is refilled
        // only after the store issued from it two fills earlier has finished READING shared memory.
        uint8_t* stg = sStage + warp * (32 * 256);
        const CUtensorMap* om = &omaps.m[owner];
        const int y = ((int)(ar_epoch & 1) * B200_MAX_RANKS + p.comm.rank) * p.slot_rows + dst_row0 + warp * 32;
#pragma unroll 1
        for (int fill = 0; fill < 4; ++fill) {
          uint32_t v[2][32];
          tmem_ld_32x32(taddr + fill * 64, v[0]);
          tmem_ld_32x32(taddr + fill * 64 + 32, v[1]);
          tmem_ld_wait();
          if (fill == 3) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) remote_arrive(lead_acc_empty0 + buf * 8);
          }
          uint8_t* box = stg + (fill & 1) * 4096;
          if (lane == 0) bulk_wait_read_1();
          __syncwarp();
#pragma unroll
          for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                oh[e] = __floats2bfloat162_rn(__uint_as_float(v[hh][q4 * 8 + 2 * e]), __uint_as_float(v[hh][q4 * 8 + 2 * e + 1]));
              const int ci = hh * 4 + q4;
              *reinterpret_cast<uint4*>(box + lane * 128 + ((ci ^ (lane & 7)) << 4)) = o;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            tma_store_2d(om, box, m2 * BN + fill * 64, y);
            tma_store_commit();
          }
        }
      } else {
        // Peer memory wants long runs: a thread's own 16-byte pieces would cross NVLink one by one.  Each warp stages
        // 32 rows x 128 features in its private shared-memory patch (16-byte chunks XOR-swizzled by row, so neither
        // side has bank conflicts) and writes it out 256 contiguous bytes per token row, two rows per instruction.
        uint8_t* stg = sStage + warp * (32 * 256);
        __nv_bfloat16* wrow = dst + (size_t)(dst_row0 + warp * 32) * p.ldo + (size_t)m2 * BN;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll 1
          for (int cc = 0; cc < 4; cc += 2) {
            uint32_t v[2][32];
            tmem_ld_32x32(taddr + half * 128 + cc * 32, v[0]);
            tmem_ld_32x32(taddr + half * 128 + cc * 32 + 32, v[1]);
            tmem_ld_wait();
            if (half == 1 && cc == 2) {
              tc_fence_before();
              __syncwarp();
              if (lane == 0) remote_arrive(lead_acc_empty0 + buf * 8);
            }
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
#pragma unroll
              for (int q4 = 0; q4 < 4; ++q4) {
                uint4 o;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e)
                  oh[e] = __floats2bfloat162_rn(__uint_as_float(v[hh][q4 * 8 + 2 * e]), __uint_as_float(v[hh][q4 * 8 + 2 * e + 1]));
                const int ci = (cc + hh) * 4 + q4;
                *reinterpret_cast<uint4*>(stg + lane * 256 + ((ci ^ (lane & 7)) << 4)) = o;
              }
            }
          }
          __syncwarp();
#pragma unroll 4
          for (int j = 0; j < 16; ++j) {
            const int r = (lane >> 4) + 2 * j, ci = lane & 15;
            const uint4 q = *reinterpret_cast<const uint4*>(stg + r * 256 + ((ci ^ (r & 7)) << 4));
            *reinterpret_cast<uint4*>(wrow + (size_t)r * p.ldo + half * 128 + ci * 8) = q;
          }
          __syncwarp();
        }
      }
      if (p.mode == 3) {
        if (!p.tma_push) {
          signal_tile(tile_i, owner, dst_row0, m2);
        } else {
          // Bulk stores complete asynchronously.  Waiting for them here would idle the warp for a link round trip per
          // tile, so a tile's flags are raised one tile late: "at most this tile's four store groups still pending"
          // means that every group of the previous tile has landed.
          if (have_prev) {
            if (lane == 0) bulk_wait_4();
            signal_tile(tile_i - 1, prev_owner, prev_row0, prev_m2);
          }
          have_prev = true;
          prev_owner = owner;
          prev_row0 = dst_row0;
          prev_m2 = m2;
        }
      }
    }
    // bulk stores still in flight belong to this warp's lane 0: drain them before the shared memory goes away, then
    // raise the last tile's flags
    if (p.mode == 3 && p.tma_push) {
      if (lane == 0) tma_store_wait_all();
      if (have_prev && !*abort_flag) signal_tile(tile_i - 1, prev_owner, prev_row0, prev_m2);
    }
  }

  // Common exit.  The pair leaves together: the leader's commits land in the peer's barriers and its MMAs read the
  // peer's shared memory, so neither CTA may retire while the other can still touch it.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    const uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  cluster_sync_all();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
  if (p.mode == 3 && threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(&p.comm.ctrl[1], 1u) + 1;
    if (done == gridDim.x) {
      p.comm.ctrl[1] = 0;
      __threadfence();
      atomicExch(&p.comm.ctrl[0], ar_epoch);
    }
  }
}

}  // namespace g2
}  // namespace b200

using namespace b200;

static int g_2cta_enabled = 1;

extern "C" void b200_gemm_2cta_enable(int on) { g_2cta_enabled = on; }
extern "C" int b200_gemm_2cta_enabled(void) { return g_2cta_enabled; }

extern "C" int b200_gemm_2cta_supported(int T, int N, int K) {
  return g_2cta_enabled && T > 0 && T % (2 * g2::BM) == 0 && N % g2::BN == 0 && K % g2::BK == 0 && K >= g2::BK;
}

// Tensor maps of the owners' data regions for the bulk-store push, cached per (regions, row length, slot size): the
// regions of a communicator never move, and encoding eight maps per launch would cost the host ~10 us.
static bool push_maps(const B200Comm& c, int ldo, g2::OutMaps* out) {
  struct Entry {
    void* data[B200_MAX_RANKS];
    int world, ldo;
    unsigned long long slot_elems;
    g2::OutMaps maps;
  };
  static std::mutex mu;
  static std::vector<Entry> cache;
  std::lock_guard<std::mutex> lock(mu);
  for (const Entry& e : cache)
    if (e.world == c.world && e.ldo == ldo && e.slot_elems == c.slot_elems &&
        memcmp(e.data, c.data, sizeof(void*) * c.world) == 0) {
      *out = e.maps;
      return true;
    }
  Entry e;
  memset(&e, 0, sizeof(e));
  e.world = c.world;
  e.ldo = ldo;
  e.slot_elems = c.slot_elems;
  const uint64_t rows = 2ull * B200_MAX_RANKS * (c.slot_elems / (unsigned long long)ldo);
  for (int r = 0; r < c.world; ++r) {
    e.data[r] = c.data[r];
    if ((reinterpret_cast<uintptr_t>(c.data[r]) & 15) ||
        !make_tmap_2d(&e.maps.m[r], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, c.data[r], rows, (uint64_t)ldo, (uint64_t)ldo * 2,
                      32, 64, CU_TENSOR_MAP_SWIZZLE_128B))
      return false;
  }
  if (cache.size() >= 16) cache.erase(cache.begin());
  cache.push_back(e);
  *out = e.maps;
  return true;
}

// X [T, K] bf16, W [N, K] bf16 -> out [T, N] bf16 (mode 0), or the reduce-scatter push of the sequence-parallel path
// (mode 3: out unused; comm, sp_rows and n_rot as in gemm_wdec_kernel.cuh), or out [T, N / 2] = silu(gate) * up for a
// W whose rows are interleaved in 128-row tiles [gate | up] (mode 4).  ag_wait: X is the gathered buffer.
extern "C" int b200_gemm_bf16_2cta(const void* W, const void* X, void* out_bf16, int T, int N, int K, int mode,
                                   const B200Comm* comm, int sp_rows, int n_rot, int ag_wait, int ag_flag_rows,
                                   unsigned long long budget_ns, int* status, cudaStream_t stream) {
  if (!b200_gemm_2cta_supported(T, N, K) || (mode != 0 && mode != 3 && mode != 4) || (mode != 3 && !out_bf16))
    return -ERR_BAD_ARG;
  if ((mode == 3 || ag_wait) && (!comm || sp_rows <= 0 || sp_rows % (2 * g2::BM))) return -ERR_BAD_ARG;
  if (ag_wait && (ag_flag_rows <= 0 || g2::BM % ag_flag_rows)) return -ERR_BAD_ARG;
  g2::Params p;
  memset(&p, 0, sizeof(p));
  p.T = T; p.N = N; p.K = K;
  p.kb_total = K / g2::BK;
  p.m2_tiles = N / g2::BN;
  p.n_tiles = T / (2 * g2::BM);
  p.ldo = mode == 4 ? N / 2 : N;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.status = status;
  p.mode = mode;
  p.n_rot = n_rot;
  p.sp_rows = sp_rows;
  p.ag_wait = ag_wait;
  p.ag_flag_rows = ag_flag_rows;
  p.budget_ns = budget_ns ? budget_ns : B200_WAIT_BUDGET_NS;
  if (comm) p.comm = *comm;
  g2::OutMaps omaps;
  memset(&omaps, 0, sizeof(omaps));
  if (mode == 3) {
    static const bool want = [] { const char* e = getenv("B200_RS_TMA"); return !(e && e[0] == '0'); }();
    if (want && comm->slot_elems % (unsigned long long)N == 0 && push_maps(*comm, N, &omaps)) {
      p.tma_push = 1;
      p.slot_rows = (int)(comm->slot_elems / (unsigned long long)N);
    }
  }
  CUtensorMap tmW, tmX;
  if (!make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, (uint64_t)K * 2, g2::BNH, g2::BK,
                    CU_TENSOR_MAP_SWIZZLE_128B) ||
      !make_tmap_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, T, K, (uint64_t)K * 2, g2::BM, g2::BK,
                    CU_TENSOR_MAP_SWIZZLE_128B))
    return -ERR_BAD_ARG;
  static b200::PerDeviceOnce once_;
  bool& configured = once_.slot();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(g2::gemm_bf16_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         g2::SMEM_TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int total = p.m2_tiles * p.n_tiles;
  int pairs = sm_count() / 2;
  if (pairs > total) pairs = total;
  g2::gemm_bf16_2cta_kernel<<<2 * pairs, g2::THREADS, g2::SMEM_TOTAL, stream>>>(tmW, tmX, omaps, p);
  return (int)cudaGetLastError();
}
