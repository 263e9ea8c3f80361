// Weight-decoding tensor-core GEMM for sm_100a:  Y[T, N] = X[T, K] * W[N, K]^T.
//
// Design (one persistent CTA per SM, 14 warps, warp-specialised):
//   * W is the UMMA "A" operand (M = 128 output features per tile) and the
//     activations are the "B" operand (N = BN tokens, 16..256), so the same
//     kernel serves prefill (BN = 256) and decode batches (BN = 16..64) while
//     the weight tile is always a full 128-row MMA.
//   * warp 4 streams raw weight bytes and bf16 activations with TMA
//     (cp.async.bulk.tensor, destination = this CTA only, never multicast);
//   * warps 6..13 decode the raw weight tile (FP8 E4M3 with one scale per
//     128x128 block) into bf16, written in the 128-byte-swizzled K-major layout
//     the tensor core reads; the quantised matrix is never expanded in HBM;
//   * warp 5 issues tcgen05.mma (kind::f16, fp32 accumulate in TMEM, two
//     accumulator buffers) and commits stage/accumulator barriers;
//   * warps 0..3 drain TMEM with tcgen05.ld and store bf16 (+residual) or fp32
//     split-K partials.
// Every mbarrier wait is bounded; on expiry the CTA records an error code and
// unwinds through the common exit (TMEM is always freed).
//
// Reference behaviour covered: FP8 block-128 weight x 16-bit activation
// projections of the Qwen path (cpp_engine/backends/cuda/kernels/qwen_half_ops.cu:988-1199,
// dequant + cublasGemmEx at :1349) and dense bf16 projections
// (cpp_engine/backends/cuda/kernels/bf16_ops.cu:30-167).
// (Kernel template and launcher; the extern "C" entry points live in gemm_wdec.cu and gemm_wdec_gguf.cu, which
// instantiate it for their weight formats so the formats compile in parallel.)
#pragma once
#include <cuda_bf16.h>
#include "per_device.h"
#include <cuda_fp8.h>
#include <cuda_fp16.h>
#include <string.h>
#include "../ptx/sm100.cuh"
#include "tma_host.h"
#include "ops.h"
#include "../comm/comm.h"

namespace b200 {

constexpr int BM = 128;      // output features per tile (UMMA M)
constexpr int BK = 64;       // K elements per pipeline stage (one 128-byte swizzle row of bf16)
constexpr int NUM_EPI_WARPS = 4;
constexpr int TMA_WARP = 4;
constexpr int MMA_WARP = 5;
constexpr int DEC_WARP0 = 6;
constexpr int NUM_DEC_WARPS = 8;
constexpr int NUM_THREADS = (DEC_WARP0 + NUM_DEC_WARPS) * 32;  // 448

// WF_FP4: E2M1 nibbles (low nibble first) with one UE8M0 scale per 32 inputs, stored tile-major as
// [m_tile][kb][128 rows x 32 code bytes | 128 rows x 2 scale bytes] (4352 bytes per stage).
// GGUF block formats keep their quantised bytes; they are only regrouped at load time so that one pipeline stage
// (128 rows x 64 inputs) is a contiguous block [128 x QB quant bytes | 128 x SB scale bytes]:
//   WF_Q8_0     QB 64 (int8), SB 4: two fp16 block scales
//   WF_Q4_K     QB 32 (low nibble = input l, high nibble = input 32 + l), SB 8: d, dmin (fp16), sc0, m0, sc1, m1 (6-bit values)
//   WF_Q2_K     QB 16 (four 2-bit codes per byte: inputs l, 32 + l of byte l & 15 ...), SB 8: d, dmin (fp16), four scale|min bytes
//   WF_IQ2_XXS  QB 16 (two original 8-byte groups of 32 inputs), SB 4: d (fp16)
//   WF_Q5_K     QB 40 (Q4_K nibbles, then two 32-bit masks holding the fifth bit of inputs l and 32 + l), SB 8 as Q4_K
//   WF_IQ3_XXS  QB 24 (16 grid indices, then the two sign/scale words of the stage's 32-input groups), SB 4: d (fp16)
//   WF_IQ1_M    QB 12 (8 low index bytes, then 4 bytes of high index bits / delta signs), SB 4: d (fp16), one byte per
//               32-input group holding its two 3-bit scales
//   WF_Q6_K     QB 48 (Q4_K-style nibbles, then per half a 64-bit word with the two high bits of input l at bits 2l),
//               SB 8: d (fp16), 2 pad bytes, four int8 scales (one per 16 inputs)
//   WF_Q3_K     QB 24 (per half a 64-bit word of 2-bit codes, then per half a 32-bit mask of the third bit),
//               SB 8: d (fp16), 2 pad bytes, four signed 6-bit scales (already minus 32) as int8
//   WF_IQ4_XS   QB 32 (the stage's two original 16-byte sub-blocks: low nibble = input l, high = input 16 + l),
//               SB 4: d (fp16), two int8 scales (already minus 32); 16-entry int8 value table
//   WF_IQ2_XS   QB 16 (eight original 16-bit codes: 9-bit grid index | 7-bit sign index << 9), SB 4: d (fp16), the two
//               scale bytes (4 bits per 16 inputs); 512 x 8 magnitude grid + 128 sign bytes
enum WFormat : int {
  WF_BF16 = 0, WF_FP8_B128 = 1, WF_FP4 = 2, WF_Q8_0 = 3, WF_Q4_K = 4, WF_Q2_K = 5, WF_IQ2_XXS = 6, WF_Q5_K = 7,
  WF_IQ3_XXS = 8, WF_IQ1_M = 9, WF_Q6_K = 10, WF_Q3_K = 11, WF_IQ4_XS = 12, WF_IQ2_XS = 13
};

__host__ __device__ constexpr int gguf_qb(int wfmt) {
  return wfmt == WF_Q8_0 ? 64 : wfmt == WF_Q4_K ? 32 : wfmt == WF_Q2_K ? 16 : wfmt == WF_IQ2_XXS ? 16
         : wfmt == WF_Q5_K ? 40 : wfmt == WF_IQ3_XXS ? 24 : wfmt == WF_IQ1_M ? 12 : wfmt == WF_Q6_K ? 48
         : wfmt == WF_Q3_K ? 24 : wfmt == WF_IQ4_XS ? 32 : wfmt == WF_IQ2_XS ? 16 : 0;
}
__host__ __device__ constexpr int gguf_sb(int wfmt) {
  return wfmt == WF_Q8_0 ? 4 : wfmt == WF_Q4_K ? 8 : wfmt == WF_Q2_K ? 8 : wfmt == WF_IQ2_XXS ? 4
         : wfmt == WF_Q5_K ? 8 : wfmt == WF_IQ3_XXS ? 4 : wfmt == WF_IQ1_M ? 4 : wfmt == WF_Q6_K ? 8 : wfmt == WF_Q3_K ? 8
         : wfmt == WF_IQ4_XS ? 4 : wfmt == WF_IQ2_XS ? 4 : 0;
}
__host__ __device__ constexpr int raw_stage_bytes(int wfmt) {
  return wfmt == WF_FP8_B128 ? 128 * 64
         : wfmt == WF_FP4    ? 128 * 32 + 128 * 2
         : gguf_qb(wfmt)     ? 128 * (gguf_qb(wfmt) + gguf_sb(wfmt))
                             : 0;
}

struct GemmParams {
  int T, N, K;
  int m_tiles, n_tiles, splits, kb_total;
  const uint8_t* w_tiled;  // FP8 only: [m_tiles][kb_total][128 rows][64 bytes], bytes pre-shuffled
  const float* scales;  // [ceil(N/128), scale_ld] fp32 (FP8 only)
  int scale_ld;
  __nv_bfloat16* out;        // [T, ldo] (splits == 1)
  float* out_f32;            // [splits, T, ldo] partials (splits > 1) or fp32 result
  const __nv_bfloat16* residual;  // optional [T, ldo], added in the epilogue (splits == 1)
  int ldo;
  int* status;
  // In-kernel split-K fix-up (splits > 1 with `out` set): every split writes its fp32 partial to
  // out_f32, then bumps tile_counters[tile]; the CTA that arrives last sums the partials in split
  // order (so the result does not depend on which CTA is last), adds the residual, stores bf16 and
  // resets the counter.  tile_counters must be zero before the first use.
  int* tile_counters;
  // Grouped mode (routed experts): work_table[i] = {group, m_tile, first row, rows (<= BN)} and *num_work entries,
  // both written on the device by the routing kernels; group g uses weights at w_tiled + g * w_group_stride
  // (bf16: rows g*N.. of the weight tensor map) and scales at scales + g * scale_group_stride.  splits == 1.
  const uint8_t* lut;        // IQ formats: codebook (256 x 8 bytes) followed by the 128-byte sign table, in global memory
  const int4* work_table;
  const int* num_work;
  size_t w_group_stride;
  size_t scale_group_stride;
  // Fused all-reduce (row-parallel GEMM under tensor parallelism).
  // ar_mode == 1 (one-shot): the epilogue pushes this rank's partial tile to every peer, waits for theirs and
  //   stores the sum; every tile crosses NVLink world-1 times per rank.
  // ar_mode == 2 (two-shot): tile w is owned by rank w % world; the others push their partial only to the owner,
  //   the owner reduces and pushes the finished tile into every rank's result region (`out` points into this
  //   rank's).  Traffic per rank is 2 (world-1)/world of the output instead of (world-1) times it.
  // ar_mode == 3 (reduce-scatter push, sequence-parallel residual): token rows are owned in contiguous shards of
  //   sp_rows rows (rank r owns rows [r*sp_rows, (r+1)*sp_rows), sp_rows % BN == 0).  The epilogue stores each
  //   partial tile - staged through shared memory so that every thread writes 16 bytes and a token row leaves as
  //   256 contiguous bytes - only into the owner's slot for source = this rank, then raises that tile's flag on
  //   the owner.  Nothing waits here: the owner's reduce + norm kernel (comm/sp_comm.cu) consumes the partials.
  //   Each partial crosses NVLink once: (world-1)/world of the output per rank.  Token tiles are visited starting
  //   with the next rank's shard (n_rot) so that at any moment the ranks write to different owners.
  int ar_mode;
  size_t result_off;   // element offset of the output inside every rank's result region (two-shot)
  unsigned long long ar_budget_ns;
  int n_rot;           // token-tile rotation: tile index = (n + n_rot) % n_tiles (0 outside the sequence-parallel modes)
  int sp_rows;         // rows per owner shard (ar_mode 3, ag_wait)
  // ag_wait (all-gather + GEMM): the activation rows of shard s != rank are pushed into this rank's X by rank s
  //   (comm/sp_comm.cu), which then raises one flag per ag_flag_rows rows in the second flag bank.  The producer
  //   warp waits for the flags of a token tile before its first TMA load of that tile; X itself is local memory.
  int ag_wait;
  int ag_flag_rows;
  B200Comm comm;
};

// Shared memory holds two rings.  The "raw" ring (SR stages) receives what TMA brings: the
// activation tile plus either the raw FP8 weight tile or, for bf16 weights, the ready-to-use
// weight tile.  The "decoded" ring (SA stages, FP8 only) holds bf16 weight tiles written by the
// decode warps.  Raw FP8 stages are small (8 KB), so the raw ring is deep enough (up to 16
// stages, >= 100 KB per SM in flight) to keep HBM busy in the weight-streaming decode regime,
// while the 16 KB decoded tiles only need enough stages to overlap decode with the MMA.
struct Work {
  int group, m_tile, row0, rows, split;
};

template <int BN>
__device__ __forceinline__ Work get_work(const GemmParams& p, int w) {
  Work k;
  if (p.work_table) {
    const int4 e = p.work_table[w];
    k.group = e.x; k.m_tile = e.y; k.row0 = e.z; k.rows = e.w; k.split = 0;
  } else {
    k.group = 0;
    k.m_tile = w % p.m_tiles;
    const int rest = w / p.m_tiles;
    int n_tile = rest % p.n_tiles + p.n_rot;
    if (n_tile >= p.n_tiles) n_tile -= p.n_tiles;
    k.split = rest / p.n_tiles;
    k.row0 = n_tile * BN;
    k.rows = min(BN, p.T - k.row0);
  }
  return k;
}

template <int BN, int WFMT>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;       // 16 KB bf16 weights (decoded, or loaded for WF_BF16)
  static constexpr int X_BYTES = BN * BK * 2;       // activations
  static constexpr int RAW_BYTES = raw_stage_bytes(WFMT) ? raw_stage_bytes(WFMT) : BM * BK;   // raw quantised tile
  // Epilogue staging for the reduce-scatter mode (two 32-token x 128-feature bf16 half-tiles), reserved only where
  // it costs no decode-regime pipeline depth: the prefill-sized tiles of the bf16 and FP8 formats.
  static constexpr int EPI_BYTES =
      ((WFMT == WF_BF16 && BN >= 128) || (WFMT == WF_FP8_B128 && BN == 128)) ? 16384 : 0;
  static constexpr int BUDGET = 232448 - 1024 /*align slack*/ - 512 /*barriers*/ - EPI_BYTES;
  static constexpr int SA = (WFMT == WF_BF16) ? 0 : 4;
  static constexpr int W_STAGE_BYTES = (WFMT == WF_BF16) ? A_BYTES : RAW_BYTES;
  static constexpr int STAGE_BYTES = W_STAGE_BYTES + X_BYTES;
  static constexpr int SR_RAW = (BUDGET - SA * A_BYTES) / STAGE_BYTES;
  static constexpr int SR = SR_RAW > 16 ? 16 : SR_RAW;
  static constexpr int TOTAL = SR * STAGE_BYTES + SA * A_BYTES + EPI_BYTES + 1024 + 512;
  // Decode warps work in GROUPS independent groups; group g owns decoded slot g and every
  // GROUPS-th k-block, so barrier/fence latency of one stage overlaps another's ALU work.
  static constexpr int GROUPS = 4;
  static constexpr int WARPS_PER_GROUP = NUM_DEC_WARPS / GROUPS;
  static_assert(SR >= 2, "pipeline needs at least two raw stages");
};

// 4 fp8 bytes stored as (w0, w2, w1, w3) -> two bf16x2 words (w0,w1), (w2,w3),
// each still scaled by 2^-120; the caller multiplies by scale * 2^120.
__device__ __forceinline__ void fp8x4_to_bf16x4_raw(uint32_t q, uint32_t& w01, uint32_t& w23) {
  w23 = (q & 0x80008000u) | ((q & 0x7F007F00u) >> 4);
  uint32_t q2 = q << 8;
  w01 = (q2 & 0x80008000u) | ((q2 & 0x7F007F00u) >> 4);
}
__device__ __forceinline__ uint32_t bf16x2_mul(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}

template <int BN, int WFMT>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_wdec_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                 GemmParams p) {
  using L = SmemLayout<BN, WFMT>;
  constexpr int S = L::SR;                       // raw ring depth
  constexpr int SA = L::SA;                      // decoded ring depth (0 for bf16 weights)
  constexpr int SAB = SA > 0 ? SA : 1;
  constexpr uint32_t TMEM_COLS = (2 * BN < 32) ? 32 : 2 * BN;
  extern __shared__ uint8_t smem_raw_base[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw_base) + 1023) &
                                             ~uintptr_t(1023));
  // bf16 weights: sA is the raw ring itself (S stages); FP8: sA is the decoded ring (SA stages)
  uint8_t* sA = smem;
  uint8_t* sX = sA + (WFMT == WF_BF16 ? S : SA) * L::A_BYTES;
  uint8_t* sRaw = sX + S * L::X_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sRaw + (WFMT == WF_BF16 ? 0 : S * L::RAW_BYTES));
  uint64_t* tma_full = bars;                  // [S]   raw stage landed
  uint64_t* empty = bars + S;                 // [S]   k-block consumed (MMA commit): raw stage and decoded slot
  uint64_t* a_full = bars + 2 * S;            // [SAB] decoded tile written
  uint64_t* acc_full = bars + 2 * S + SAB;       // [2]
  uint64_t* acc_empty = bars + 2 * S + SAB + 2;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + SAB + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* fix_last = const_cast<int*>(abort_flag) + 1;   // split-K fix-up: "this CTA finishes the tile"
  volatile int* epi_abort = reinterpret_cast<volatile int*>(fix_last + 1);  // written by epilogue threads only
  __nv_bfloat16* sEpi = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(bars) + 512);  // L::EPI_BYTES

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(&tma_full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < SAB; ++s) {
      mbar_init(&a_full[s], L::WARPS_PER_GROUP);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&acc_full[b], 1);
      mbar_init(&acc_empty[b], NUM_EPI_WARPS * 32);
    }
    *abort_flag = 0;
    *epi_abort = 0;
    mbar_fence_init();
  }
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if (warp == TMA_WARP && lane == 0) {
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmX);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t ar_epoch_at_entry = p.ar_mode ? p.comm.ctrl[0] + 1 : 0;

  const int total_work = p.work_table ? *p.num_work : p.m_tiles * p.n_tiles * p.splits;
  const int kb_per_split = (p.kb_total + p.splits - 1) / p.splits;

  if (warp == TMA_WARP) {
    // ------------------------------------------------------------ TMA producer
    // The whole warp walks the tile list (so that its lanes can poll the all-gather flags of a tile side by side);
    // lane 0 alone drives the pipeline.  Loop exits are taken on values broadcast from lane 0.
    const uint32_t ag_epoch = p.ag_wait ? p.comm.ctrl[0] : 0;   // the gather kernel that ran before this one
    // once any kernel has recorded an expired wait the step is lost: do not spend the budget again
    const uint64_t ag_budget = (p.ag_wait && *reinterpret_cast<volatile int*>(p.status) == 0) ? p.ar_budget_ns : 1000;
    uint32_t it = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x) {
      int stop = (lane == 0) ? *abort_flag : 0;
      stop = __shfl_sync(0xffffffffu, stop, 0);
      if (stop) break;
      const Work wk = get_work<BN>(p, w);
      if (p.ag_wait) {
        const int src = wk.row0 / p.sp_rows;
        if (src != p.comm.rank) {
          const int first = (wk.row0 - src * p.sp_rows) / p.ag_flag_rows;
          const int cnt = (wk.rows + p.ag_flag_rows - 1) / p.ag_flag_rows;
          const uint32_t* fl = p.comm.flags2[p.comm.rank] +
                               ((size_t)(ag_epoch & 1) * B200_MAX_RANKS + src) * B200_FLAGS_PER_SLOT + first;
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
        const int m_tile = wk.m_tile;
        const int kb0 = wk.split * kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + kb_per_split);
        const uint8_t* wbase = p.w_tiled + (size_t)wk.group * p.w_group_stride;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1)) {
            atomicExch(p.status, ERR_WAIT_STAGE);
            *abort_flag = 1;
            failed = 1;
            break;
          }
          if (WFMT == WF_BF16) {
            mbar_expect_tx(&tma_full[s], L::A_BYTES + L::X_BYTES);
            tma_load_2d(sA + s * L::A_BYTES, &tmW, &tma_full[s], kb * BK, wk.group * p.N + m_tile * BM);
          } else {
            // FP8 weights are stored tile-major: one contiguous 8 KB block per (m_tile, kb)
            mbar_expect_tx(&tma_full[s], L::RAW_BYTES + L::X_BYTES);
            bulk_load(sRaw + s * L::RAW_BYTES,
                      wbase + ((size_t)m_tile * p.kb_total + kb) * L::RAW_BYTES, L::RAW_BYTES, &tma_full[s]);
          }
          tma_load_2d(sX + s * L::X_BYTES, &tmX, &tma_full[s], kb * BK, wk.row0);
        }
      }
      failed = __shfl_sync(0xffffffffu, failed, 0);
      if (failed) break;
    }
  } else if (warp == MMA_WARP) {
    // -------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN);
      uint32_t it = 0;
      uint32_t tile_i = 0;
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x, ++tile_i) {
        const int split = get_work<BN>(p, w).split;
        const int kb0 = split * kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + kb_per_split);
        const int buf = tile_i & 1;
        const uint32_t acc_ph = (tile_i >> 1) & 1;
        if (!mbar_wait(&acc_empty[buf], acc_ph ^ 1)) {
          atomicExch(p.status, ERR_WAIT_ACC);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        bool failed = false;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          if (!mbar_wait(&tma_full[s], ph)) {
            atomicExch(p.status, ERR_WAIT_TMA);
            failed = true;
            break;
          }
          const int sa = (WFMT == WF_BF16) ? s : (int)(it % SAB);
          if (WFMT != WF_BF16) {
            if (!mbar_wait(&a_full[sa], (it / SAB) & 1)) {
              atomicExch(p.status, ERR_WAIT_DEQUANT);
              failed = true;
              break;
            }
          }
          tc_fence_after();
          const uint64_t da = umma_desc_sw128(sA + sa * L::A_BYTES);
          const uint64_t db = umma_desc_sw128(sX + s * L::X_BYTES);
#pragma unroll
          for (int k = 0; k < BK / 16; ++k) {
            // advance 16 bf16 = 32 bytes inside the swizzle row: +2 in 16-byte units
            umma_bf16_ss(tmem_d, da + 2 * k, db + 2 * k, idesc, (kb > kb0 || k > 0) ? 1u : 0u);
          }
          // One commit per k-block frees the raw stage for the producer and, SA k-blocks later, the
          // decoded slot for the decode warps (they wait on the same barrier): tcgen05.commit occupies
          // the tensor pipe for a few hundred cycles, so a second commit per k-block would cap the rate.
          umma_commit(&empty[s]);
        }
        if (failed) {
          *abort_flag = 1;
          break;
        }
        umma_commit(&acc_full[buf]);
      }
    }
  } else if (warp >= DEC_WARP0) {
    // ------------------------------------------------- weight decode (FP8 -> bf16)
    if constexpr (WFMT != WF_BF16) {
      constexpr int G = L::GROUPS;
      static_assert(G == SAB, "one decode group per decoded slot");
      // A group's parity wait on raw stage it % S assumes k-block it - S has landed; the only ordering a group has
      // with the producer is through its own previous k-block it - G, so the ring must hold at least G stages.
      static_assert(S >= G, "raw ring shallower than the decode groups' look-ahead");
      constexpr int WPG = L::WARPS_PER_GROUP;
      constexpr int GT = WPG * 32;             // threads per group
      const int dw = warp - DEC_WARP0;
      const int grp = dw / WPG;
      const int d = (dw % WPG) * 32 + lane;    // 0..GT-1
      uint32_t it = 0;
      for (int w = blockIdx.x; w < total_work && !*abort_flag; w += gridDim.x) {
        const Work wk = get_work<BN>(p, w);
        const int m_tile = wk.m_tile;
        const int kb0 = wk.split * kb_per_split;
        const int kb1 = min(p.kb_total, kb0 + kb_per_split);
        // FP8: block scales of this tile's K range, fetched once per tile and spread over the lanes
        // (lane l holds entries l, l+32, ...): a per-stage global load would put an L2 round trip
        // on the critical path of every stage.
        const int sc_lo = kb0 >> 1;
        float my_sc[8];
        if constexpr (WFMT == WF_FP8_B128) {
          const float* srow = p.scales + (size_t)wk.group * p.scale_group_stride + (size_t)m_tile * p.scale_ld;
          const int nsc = (kb1 > kb0) ? (((kb1 - 1) >> 1) - sc_lo + 1) : 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int idx = j * 32 + lane;
            my_sc[j] = (idx < nsc) ? __ldg(srow + sc_lo + idx) * 0x1p120f : 0.f;
          }
        }
        bool failed = false;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          if ((int)(it % G) != grp) continue;
          const int s = it % S;
          const uint32_t ph = (it / S) & 1;
          uint32_t scw = 0;
          if constexpr (WFMT == WF_FP8_B128) {
            const int si = (kb >> 1) - sc_lo;
            float scv = my_sc[0];
#pragma unroll
            for (int j = 1; j < 8; ++j) scv = (si >> 5) == j ? my_sc[j] : scv;
            const float sc = __shfl_sync(0xffffffffu, scv, si & 31);
            __nv_bfloat162 sc2 = __float2bfloat162_rn(sc);
            scw = *reinterpret_cast<uint32_t*>(&sc2);
          }
          bool ok = mbar_wait(&tma_full[s], ph);
          if (it >= (uint32_t)SAB) {
            // decoded slot `grp` was last read by the MMAs of k-block it - SA
            const uint32_t prev = it - SAB;
            ok = ok && mbar_wait(&empty[prev % S], (prev / S) & 1);
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            if (lane == 0) atomicExch(p.status, ERR_WAIT_TMA);
            failed = true;
            break;
          }
          tc_fence_after();
          const uint8_t* raw = sRaw + s * L::RAW_BYTES;
          uint8_t* A = sA + grp * L::A_BYTES;
          if constexpr (WFMT == WF_FP8_B128) {
            constexpr int REPS = (BM * 4) / GT;      // 16-byte chunks (16 values) per thread per stage
            uint4 q[REPS];
#pragma unroll
            for (int rep = 0; rep < REPS; ++rep) {
              const int i = d + rep * GT;
              const int rr = i >> 2;
              q[rep] = *reinterpret_cast<const uint4*>(raw + rr * BK + (((i & 3) ^ ((rr >> 1) & 3)) << 4));
            }
#pragma unroll
            for (int rep = 0; rep < REPS; ++rep) {
              const int i = d + rep * GT;
              const int r = i >> 2, c = i & 3;
              uint4 o0, o1;
              fp8x4_to_bf16x4_raw(q[rep].x, o0.x, o0.y);
              fp8x4_to_bf16x4_raw(q[rep].y, o0.z, o0.w);
              fp8x4_to_bf16x4_raw(q[rep].z, o1.x, o1.y);
              fp8x4_to_bf16x4_raw(q[rep].w, o1.z, o1.w);
              o0.x = bf16x2_mul(o0.x, scw); o0.y = bf16x2_mul(o0.y, scw);
              o0.z = bf16x2_mul(o0.z, scw); o0.w = bf16x2_mul(o0.w, scw);
              o1.x = bf16x2_mul(o1.x, scw); o1.y = bf16x2_mul(o1.y, scw);
              o1.z = bf16x2_mul(o1.z, scw); o1.w = bf16x2_mul(o1.w, scw);
              uint8_t* rowp = A + (r >> 3) * 1024 + (r & 7) * 128;
              const int sw = r & 7;
              *reinterpret_cast<uint4*>(rowp + (((2 * c) ^ sw) << 4)) = o0;
              *reinterpret_cast<uint4*>(rowp + (((2 * c + 1) ^ sw) << 4)) = o1;
            }
          } else if constexpr (WFMT == WF_FP4) {
            // 128 rows x 32 code bytes, then 128 x 2 scale bytes; a 16-byte chunk = 32 values = one scale group.
            constexpr int REPS = (BM * 2) / GT;
            const uint8_t* sc_bytes = raw + BM * 32;
#pragma unroll
            for (int rep = 0; rep < REPS; ++rep) {
              const int i = d + rep * GT;
              const int r = i >> 1, hh = i & 1;       // row, which half of the 64-wide K tile
              const uint4 qv = *reinterpret_cast<const uint4*>(raw + r * 32 + hh * 16);
              // The code bits placed at exponent/mantissa positions of a bf16 read as value * 2^-126, so the
              // multiplier is 2^(e-127) * 2^126 = 2^(e-1): a bf16 with biased exponent e + 126, built directly.
              const uint32_t e = sc_bytes[r * 2 + hh];
              const uint32_t s1 = min(e + 126u, 254u) << 7;
              const uint32_t sw2 = s1 | (s1 << 16);
              const uint32_t qq[4] = {qv.x, qv.y, qv.z, qv.w};
              uint8_t* rowp = A + (r >> 3) * 1024 + (r & 7) * 128;
              const int sw = r & 7;
#pragma unroll
              for (int wd = 0; wd < 4; ++wd) {        // 4 bytes = 8 values = one 16-byte output chunk
                uint4 o;
                uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                  const uint32_t by = (qq[wd] >> (8 * b)) & 0xFFu;
                  const uint32_t t = by | (by << 12);   // low nibble at bits 0..3, high nibble at bits 16..19
                  const uint32_t v = ((t & 0x00070007u) << 6) | ((t & 0x00080008u) << 12);
                  ow[b] = bf16x2_mul(v, sw2);
                }
                *reinterpret_cast<uint4*>(rowp + (((hh * 4 + wd) ^ sw) << 4)) = o;
              }
            }
          }
          else if constexpr (gguf_qb(WFMT) != 0) {
            // one unit = (row, half of the 64-wide K tile) = 32 inputs -> 32 bf16 = four 16-byte chunks
            constexpr int QB = gguf_qb(WFMT), SB = gguf_sb(WFMT);
            const uint8_t* sreg = raw + BM * QB;
#pragma unroll 1
            for (int i = d; i < BM * 2; i += GT) {
              const int r = i >> 1, hh = i & 1;
              const uint8_t* qrow = raw + r * QB;
              const uint8_t* srow = sreg + r * SB;
              float v[32];
              if constexpr (WFMT == WF_Q8_0) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow + 2 * hh));
                const int4 a = *reinterpret_cast<const int4*>(qrow + hh * 32), b = *reinterpret_cast<const int4*>(qrow + hh * 32 + 16);
                const int w8[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int e = 0; e < 32; ++e) v[e] = dd * (float)(int8_t)((w8[e >> 2] >> (8 * (e & 3))) & 0xFF);
              } else if constexpr (WFMT == WF_Q4_K) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const float dm = __half2float(*reinterpret_cast<const __half*>(srow + 2));
                const float sc = dd * (float)srow[4 + 2 * hh], mn = dm * (float)srow[5 + 2 * hh];
                const int4 a = *reinterpret_cast<const int4*>(qrow), b = *reinterpret_cast<const int4*>(qrow + 16);
                const int w8[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const int by = (w8[e >> 2] >> (8 * (e & 3))) & 0xFF;
                  v[e] = sc * (float)(hh ? (by >> 4) : (by & 15)) - mn;
                }
              } else if constexpr (WFMT == WF_Q2_K) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const float dm = __half2float(*reinterpret_cast<const __half*>(srow + 2));
                const int4 a = *reinterpret_cast<const int4*>(qrow);
                const int w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const int by = (w4[(e & 15) >> 2] >> (8 * (e & 3))) & 0xFF;
                  const int nib = e < 16 ? (by & 15) : (by >> 4);
                  const int sb = srow[4 + 2 * hh + (e >> 4)];
                  v[e] = dd * (float)(sb & 15) * (float)((nib >> (2 * hh)) & 3) - dm * (float)(sb >> 4);
                }
              } else if constexpr (WFMT == WF_Q5_K) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const float dm = __half2float(*reinterpret_cast<const __half*>(srow + 2));
                const float sc = dd * (float)srow[4 + 2 * hh], mn = dm * (float)srow[5 + 2 * hh];
                const uint2 a0 = *reinterpret_cast<const uint2*>(qrow), a1 = *reinterpret_cast<const uint2*>(qrow + 8),
                            a2 = *reinterpret_cast<const uint2*>(qrow + 16), a3 = *reinterpret_cast<const uint2*>(qrow + 24);
                const uint32_t w8[8] = {a0.x, a0.y, a1.x, a1.y, a2.x, a2.y, a3.x, a3.y};
                const uint32_t hm = *reinterpret_cast<const uint32_t*>(qrow + 32 + 4 * hh);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const uint32_t by = (w8[e >> 2] >> (8 * (e & 3))) & 0xFF;
                  const uint32_t q5 = (hh ? (by >> 4) : (by & 15)) | (((hm >> e) & 1u) << 4);
                  v[e] = sc * (float)q5 - mn;
                }
              } else if constexpr (WFMT == WF_IQ3_XXS) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const uint2 gi = *reinterpret_cast<const uint2*>(qrow + hh * 8);
                const uint32_t aux = *reinterpret_cast<const uint32_t*>(qrow + 16 + hh * 4);
                const float db = dd * (0.5f + (float)(aux >> 28)) * 0.5f;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint32_t two = ((g < 2 ? gi.x : gi.y) >> (16 * (g & 1))) & 0xFFFF;
                  const uint32_t g0 = __ldg(reinterpret_cast<const uint32_t*>(p.lut) + (two & 0xFF));
                  const uint32_t g1 = __ldg(reinterpret_cast<const uint32_t*>(p.lut) + (two >> 8));
                  const uint32_t sg = __ldg(p.lut + 1024 + ((aux >> (7 * g)) & 0x7F));
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const uint32_t gv = ((e < 4 ? g0 : g1) >> (8 * (e & 3))) & 0xFF;
                    v[g * 8 + e] = ((sg >> e) & 1) ? -db * (float)gv : db * (float)gv;
                  }
                }
              } else if constexpr (WFMT == WF_IQ1_M) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const uint32_t ql = *reinterpret_cast<const uint32_t*>(qrow + hh * 4);
                const uint32_t qh = *reinterpret_cast<const uint32_t*>(qrow + 8) >> (16 * hh);
                const uint32_t sby = srow[2 + hh];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint32_t nib = (qh >> (4 * g)) & 0xF;
                  const uint32_t idx = ((ql >> (8 * g)) & 0xFF) | ((nib & 7) << 8);
                  const float dl = dd * (float)(2 * ((sby >> (3 * (g >> 1))) & 7) + 1);
                  const float delta = (nib & 8) ? -0.125f : 0.125f;
                  const uint2 gr = __ldg(reinterpret_cast<const uint2*>(p.lut) + idx);
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const int gv = (int)(int8_t)(((e < 4 ? gr.x : gr.y) >> (8 * (e & 3))) & 0xFF);
                    v[g * 8 + e] = dl * ((float)gv + delta);
                  }
                }
              } else if constexpr (WFMT == WF_Q6_K) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const float s0 = dd * (float)(int8_t)srow[4 + 2 * hh], s1 = dd * (float)(int8_t)srow[5 + 2 * hh];
                const int4 a = *reinterpret_cast<const int4*>(qrow), b = *reinterpret_cast<const int4*>(qrow + 16);
                const int w8[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
                const uint2 hb = *reinterpret_cast<const uint2*>(qrow + 32 + 8 * hh);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const int by = (w8[e >> 2] >> (8 * (e & 3))) & 0xFF;
                  const int hi = ((e < 16 ? hb.x : hb.y) >> (2 * (e & 15))) & 3;
                  const int q6 = (hh ? (by >> 4) : (by & 15)) | (hi << 4);
                  v[e] = (e < 16 ? s0 : s1) * (float)(q6 - 32);
                }
              } else if constexpr (WFMT == WF_Q3_K) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const float s0 = dd * (float)(int8_t)srow[4 + 2 * hh], s1 = dd * (float)(int8_t)srow[5 + 2 * hh];
                const uint2 lo = *reinterpret_cast<const uint2*>(qrow + 8 * hh);
                const uint32_t hm = *reinterpret_cast<const uint32_t*>(qrow + 16 + 4 * hh);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const int q = (int)(((e < 16 ? lo.x : lo.y) >> (2 * (e & 15))) & 3) - (((hm >> e) & 1) ? 0 : 4);
                  v[e] = (e < 16 ? s0 : s1) * (float)q;
                }
              } else if constexpr (WFMT == WF_IQ4_XS) {
                const float dl = __half2float(*reinterpret_cast<const __half*>(srow)) * (float)(int8_t)srow[2 + hh];
                const int4 a = *reinterpret_cast<const int4*>(qrow + 16 * hh);
                const int w4[4] = {a.x, a.y, a.z, a.w};
                const uint2 kv0 = __ldg(reinterpret_cast<const uint2*>(p.lut)), kv1 = __ldg(reinterpret_cast<const uint2*>(p.lut) + 1);
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                  const int by = (w4[(e & 15) >> 2] >> (8 * (e & 3))) & 0xFF;
                  const int nib = e < 16 ? (by & 15) : (by >> 4);
                  const uint32_t word = (nib & 8) ? ((nib & 4) ? kv1.y : kv1.x) : ((nib & 4) ? kv0.y : kv0.x);
                  v[e] = dl * (float)(int8_t)((word >> (8 * (nib & 3))) & 0xFF);
                }
              } else if constexpr (WFMT == WF_IQ2_XS) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow)) * 0.25f;
                const uint2 qw = *reinterpret_cast<const uint2*>(qrow + hh * 8);
                const uint32_t sby = srow[2 + hh];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint32_t code = ((g < 2 ? qw.x : qw.y) >> (16 * (g & 1))) & 0xFFFF;
                  const float db = dd * (0.5f + (float)((sby >> (4 * (g >> 1))) & 0xF));
                  const uint2 gr = __ldg(reinterpret_cast<const uint2*>(p.lut) + (code & 511));
                  const uint32_t sg = __ldg(p.lut + 4096 + (code >> 9));
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const uint32_t gv = ((e < 4 ? gr.x : gr.y) >> (8 * (e & 3))) & 0xFF;
                    v[g * 8 + e] = ((sg >> e) & 1) ? -db * (float)gv : db * (float)gv;
                  }
                }
              } else if constexpr (WFMT == WF_IQ2_XXS) {
                const float dd = __half2float(*reinterpret_cast<const __half*>(srow));
                const uint2 qw = *reinterpret_cast<const uint2*>(qrow + hh * 8);
                const float db = dd * (0.5f + (float)(qw.y >> 28)) * 0.25f;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                  const uint2 gr = __ldg(reinterpret_cast<const uint2*>(p.lut) + ((qw.x >> (8 * g)) & 0xFF));
                  const uint32_t sg = __ldg(p.lut + 2048 + ((qw.y >> (7 * g)) & 0x7F));
#pragma unroll
                  for (int e = 0; e < 8; ++e) {
                    const uint32_t gv = ((e < 4 ? gr.x : gr.y) >> (8 * (e & 3))) & 0xFF;
                    v[g * 8 + e] = ((sg >> e) & 1) ? -db * (float)gv : db * (float)gv;
                  }
                }
              }
              uint8_t* rowp = A + (r >> 3) * 1024 + (r & 7) * 128;
              const int sw = r & 7;
#pragma unroll
              for (int wd = 0; wd < 4; ++wd) {
                uint4 o;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(v[wd * 8 + 2 * e], v[wd * 8 + 2 * e + 1]);
                *reinterpret_cast<uint4*>(rowp + (((hh * 4 + wd) ^ sw) << 4)) = o;
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) mbar_arrive(&a_full[grp]);
        }
        if (failed) {
          *abort_flag = 1;
          break;
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue
    uint32_t tile_i = 0;
    const int row_in_tile = warp * 32 + lane;  // TMEM lane == output feature within the tile
    const uint32_t ar_epoch = p.ar_mode ? p.comm.ctrl[0] + 1 : 0;   // read before any CTA can finish
    // Modes whose epilogue uses a named barrier must leave the loop together: the decision to stop is
    // taken from epi_abort, which only epilogue threads write and always before a barrier.
    const bool sync_mode = p.ar_mode != 0 || (p.splits > 1 && p.out != nullptr);
    for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++tile_i) {
      if (sync_mode) {
        if (threadIdx.x == 0 && *abort_flag) *epi_abort = 1;
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*epi_abort) break;
      } else if (*abort_flag) {
        break;
      }
      const Work wk = get_work<BN>(p, w);
      const int m_tile = wk.m_tile;
      const int split = wk.split;
      const int n_tile = wk.row0 / BN;     // dense mode only (fix-up counters, all-reduce flags)
      const int buf = tile_i & 1;
      const uint32_t acc_ph = (tile_i >> 1) & 1;
      bool ok = mbar_wait(&acc_full[buf], acc_ph);
      ok = __all_sync(0xffffffffu, ok);
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
      tc_fence_after();
      const int f = m_tile * BM + row_in_tile;
      const bool f_ok = f < p.N;
      const uint32_t taddr = tmem_base + (uint32_t(warp * 32) << 16) + buf * BN;
      constexpr int CH = BN >= 32 ? 32 : 16;
      if (p.ar_mode == 3) {
        // ---- reduce-scatter push: partial tile -> the owner's slot for source = this rank ----------------------
        if constexpr (L::EPI_BYTES > 0) {
          const B200Comm& cm = p.comm;
          const int parity = ar_epoch & 1;
          const int owner = wk.row0 / p.sp_rows;
          const int local_row0 = wk.row0 - owner * p.sp_rows;
          __nv_bfloat16* dst_slot = reinterpret_cast<__nv_bfloat16*>(cm.data[owner]) +
                                    ((size_t)parity * B200_MAX_RANKS + cm.rank) * cm.slot_elems;
          const int et = threadIdx.x;            // 0..127 inside the epilogue group
          const int chunk = et & 15, trow = et >> 4;
          const int fc = m_tile * BM + chunk * 8;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            uint32_t v[32];
            tmem_ld_32x32(taddr + c0, v);
            tmem_ld_wait();
            __nv_bfloat16* st = sEpi + ((c0 >> 5) & 1) * (32 * BM);
#pragma unroll
            for (int j = 0; j < 32; ++j) st[j * BM + row_in_tile] = __float2bfloat16(__uint_as_float(v[j]));
            if (c0 + 32 >= BN) {
              tc_fence_before();
              mbar_arrive(&acc_empty[buf]);      // the accumulator is in registers / shared memory now
            }
            // One barrier per half-tile: it orders this half's writes before its reads, and (a thread passes it
            // only after its reads of the previous half) the reads of a half before its rewrite two steps later.
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (fc < p.N) {
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int tt = c0 + trow + 8 * i;
                if (tt < wk.rows) {
                  const uint4 q = *reinterpret_cast<const uint4*>(st + (trow + 8 * i) * BM + chunk * 8);
                  *reinterpret_cast<uint4*>(dst_slot + (size_t)(local_row0 + tt) * p.ldo + fc) = q;
                }
              }
            }
          }
          __threadfence_system();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et == 0) {
            const int tile_local = (local_row0 / BN) * p.m_tiles + m_tile;
            st_release_sys(cm.flags[owner] + ((size_t)parity * B200_MAX_RANKS + cm.rank) * B200_FLAGS_PER_SLOT + tile_local,
                           ar_epoch);
          }
        }
        continue;
      }
      if (p.ar_mode != 0) {
        // ---- fused all-reduce over peer memory --------------------------------------------------
        // The accumulator is first written as bf16 into this rank's own slot (a thread owns one feature, so these
        // are 2-byte stores, 64 bytes wide per warp: fine locally, far too fine for NVLink).  Everything that
        // crosses NVLink or is summed afterwards uses the transposed mapping: 16 threads cover the 256 contiguous
        // bytes of one token row with 16-byte accesses, several rows in flight per thread.
        const B200Comm& cm = p.comm;
        const int parity = ar_epoch & 1;
        const bool two_shot = p.ar_mode == 2;
        const int owner = two_shot ? (w % cm.world) : cm.rank;
        const bool reduce_here = owner == cm.rank;
        const size_t slot_elems = cm.slot_elems;
        const size_t my_slot = ((size_t)parity * B200_MAX_RANKS + cm.rank) * slot_elems;
        __nv_bfloat16* mine_slot = reinterpret_cast<__nv_bfloat16*>(cm.data[cm.rank]) + my_slot;
        const int et = threadIdx.x;            // 0..127 inside the epilogue group
        const int chunk = et & 15, trow = et >> 4;
        const int fc = m_tile * BM + chunk * 8;
        // pass 1a: accumulator -> my slot; after it the TMEM buffer can be handed back to the MMA warp
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += CH) {
          uint32_t v[32];
          if (CH == 32) {
            tmem_ld_32x32(taddr + c0, v);
          } else {
            uint32_t v16[16];
            tmem_ld_32x16(taddr + c0, v16);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = v16[j];
          }
          tmem_ld_wait();
          const int t0 = wk.row0 + c0;
          if (f_ok) {
            __nv_bfloat16* dst = mine_slot + (size_t)t0 * p.ldo + f;
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (c0 + j < wk.rows) dst[(size_t)j * p.ldo] = __float2bfloat16(__uint_as_float(v[j]));
          }
        }
        tc_fence_before();
        mbar_arrive(&acc_empty[buf]);
        __threadfence_block();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // pass 1b: push my partial to every peer (one-shot) or to the tile's owner (two-shot), 4 rows per thread in flight
        if (fc < p.N && !(two_shot && reduce_here)) {
          for (int r = 0; r < cm.world; ++r) {
            if (r == cm.rank || (two_shot && r != owner)) continue;
            __nv_bfloat16* peer_slot = reinterpret_cast<__nv_bfloat16*>(cm.data[r]) + my_slot;
            for (int tt = trow; tt < wk.rows; tt += 32) {
              uint4 q[4];
#pragma unroll
              for (int u = 0; u < 4; ++u)
                if (tt + 8 * u < wk.rows)
                  q[u] = __ldcg(reinterpret_cast<const uint4*>(mine_slot + (size_t)(wk.row0 + tt + 8 * u) * p.ldo + fc));
#pragma unroll
              for (int u = 0; u < 4; ++u)
                if (tt + 8 * u < wk.rows)
                  *reinterpret_cast<uint4*>(peer_slot + (size_t)(wk.row0 + tt + 8 * u) * p.ldo + fc) = q[u];
            }
          }
          __threadfence_system();
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        // flags: tell the consumer(s) that my partial is there; whoever reduces waits for everyone else's
        if (et < cm.world && et != cm.rank) {
          if (!two_shot || (et == owner && !reduce_here))
            st_release_sys(cm.flags[et] + ((size_t)parity * B200_MAX_RANKS + cm.rank) * B200_FLAGS_PER_SLOT + w, ar_epoch);
          if (reduce_here) {
            const uint32_t* mine = cm.flags[cm.rank] + ((size_t)parity * B200_MAX_RANKS + et) * B200_FLAGS_PER_SLOT + w;
            if (!wait_flag_ge(mine, ar_epoch, p.ar_budget_ns)) {
              atomicExch(p.status, ERR_WAIT_PEER);
              *abort_flag = 1;
              *epi_abort = 1;
            }
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*epi_abort) break;
        if (reduce_here && fc < p.N) {
          // pass 2: sum the bf16 partials of all ranks in rank order (+ residual); every rank that reduces a tile
          // reads the same bits in the same order, so the result is identical everywhere.  Two-shot: the owner also
          // stores the finished rows straight into every peer's result region.
          const __nv_bfloat16* slots0 = reinterpret_cast<const __nv_bfloat16*>(cm.data[cm.rank]) +
                                        (size_t)parity * B200_MAX_RANKS * slot_elems;
          constexpr int ROWS = 4;   // token rows in flight per thread
          for (int tt = trow; tt < wk.rows; tt += 8 * ROWS) {
            float acc[ROWS][8];
            size_t off[ROWS];
            bool live[ROWS];
#pragma unroll
            for (int u = 0; u < ROWS; ++u) {
              live[u] = tt + 8 * u < wk.rows;
              off[u] = (size_t)(wk.row0 + tt + 8 * u) * p.ldo + fc;
#pragma unroll
              for (int e = 0; e < 8; ++e) acc[u][e] = 0.f;
            }
            if (p.residual) {
              uint4 q[ROWS];
#pragma unroll
              for (int u = 0; u < ROWS; ++u)
                if (live[u]) q[u] = *reinterpret_cast<const uint4*>(p.residual + off[u]);
#pragma unroll
              for (int u = 0; u < ROWS; ++u) {
                if (!live[u]) continue;
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&q[u]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 fv = __bfloat1622float2(h2[e]);
                  acc[u][2 * e] = fv.x;
                  acc[u][2 * e + 1] = fv.y;
                }
              }
            }
#pragma unroll 2
            for (int r = 0; r < cm.world; ++r) {
              uint4 q[ROWS];
              const __nv_bfloat16* sl = slots0 + (size_t)r * slot_elems;
#pragma unroll
              for (int u = 0; u < ROWS; ++u)
                if (live[u]) q[u] = __ldcg(reinterpret_cast<const uint4*>(sl + off[u]));
#pragma unroll
              for (int u = 0; u < ROWS; ++u) {
                if (!live[u]) continue;
                const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&q[u]);
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const float2 fv = __bfloat1622float2(h2[e]);
                  acc[u][2 * e] += fv.x;
                  acc[u][2 * e + 1] += fv.y;
                }
              }
            }
#pragma unroll
            for (int u = 0; u < ROWS; ++u) {
              if (!live[u]) continue;
              uint4 o;
              __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
              for (int e = 0; e < 4; ++e) oh[e] = __floats2bfloat162_rn(acc[u][2 * e], acc[u][2 * e + 1]);
              *reinterpret_cast<uint4*>(p.out + off[u]) = o;
              if (two_shot) {
                for (int r = 0; r < cm.world; ++r)
                  if (r != cm.rank)
                    *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(cm.result[r]) + p.result_off + off[u]) = o;
              }
            }
          }
        }
        if (two_shot && reduce_here) {
          __threadfence_system();
          asm volatile("bar.sync 1, 128;" ::: "memory");
          if (et < cm.world && et != cm.rank)
            st_release_sys(cm.flags2[et] + ((size_t)parity * B200_MAX_RANKS + cm.rank) * B200_FLAGS_PER_SLOT + w, ar_epoch);
        }
        continue;
      }
#pragma unroll 1
      for (int c0 = 0; c0 < BN; c0 += CH) {
        uint32_t v[32];
        if (CH == 32) {
          tmem_ld_32x32(taddr + c0, v);
        } else {
          uint32_t v16[16];
          tmem_ld_32x16(taddr + c0, v16);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = v16[j];
        }
        tmem_ld_wait();
        const int t0 = wk.row0 + c0;
        if (f_ok) {
          if (p.splits > 1 || p.out == nullptr) {
            float* o = p.out_f32 + ((size_t)split * p.T + t0) * p.ldo + f;
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (c0 + j < wk.rows) o[(size_t)j * p.ldo] = __uint_as_float(v[j]);
          } else if (p.residual) {
            const __nv_bfloat16* r = p.residual + (size_t)t0 * p.ldo + f;
            __nv_bfloat16* o = p.out + (size_t)t0 * p.ldo + f;
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (c0 + j < wk.rows)
                o[(size_t)j * p.ldo] =
                    __float2bfloat16(__uint_as_float(v[j]) + __bfloat162float(r[(size_t)j * p.ldo]));
          } else {
            __nv_bfloat16* o = p.out + (size_t)t0 * p.ldo + f;
#pragma unroll
            for (int j = 0; j < CH; ++j)
              if (c0 + j < wk.rows) o[(size_t)j * p.ldo] = __float2bfloat16(__uint_as_float(v[j]));
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
      if (p.splits > 1 && p.out != nullptr) {
        // ---- split-K fix-up by the last-arriving CTA of this output tile
        __threadfence();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        const int tile_id = n_tile * p.m_tiles + m_tile;
        if (threadIdx.x == 0) {
          const int prev = atomicAdd(&p.tile_counters[tile_id], 1);
          *fix_last = (prev == p.splits - 1);
          if (prev == p.splits - 1) p.tile_counters[tile_id] = 0;
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (*fix_last && f_ok) {
          __threadfence();
          const int t_lo = wk.row0;
          const int t_hi = wk.row0 + wk.rows;
          for (int t = t_lo; t < t_hi; ++t) {
            const size_t off = (size_t)t * p.ldo + f;
            float acc = p.residual ? __bfloat162float(p.residual[off]) : 0.f;
            for (int sp = 0; sp < p.splits; ++sp)
              acc += __ldcg(p.out_f32 + (size_t)sp * p.T * p.ldo + off);
            p.out[off] = __float2bfloat16(acc);
          }
        }
        asm volatile("bar.sync 1, 128;" ::: "memory");   // fix_last is rewritten by the next tile
      }
    }
  }

  if (warp < NUM_EPI_WARPS && p.ar_mode == 2 && !*abort_flag) {
    // two-shot: the tiles this CTA handed to other owners must have come back before the grid may finish
    const B200Comm& cm = p.comm;
    const uint32_t epoch = ar_epoch_at_entry;
    const int parity = epoch & 1;
    int n = 0;
    for (int w = blockIdx.x; w < total_work; w += gridDim.x, ++n) {
      const int owner = w % cm.world;
      if (owner == cm.rank || (n % 128) != (int)threadIdx.x) continue;
      const uint32_t* fl = cm.flags2[cm.rank] + ((size_t)parity * B200_MAX_RANKS + owner) * B200_FLAGS_PER_SLOT + w;
      if (!wait_flag_ge(fl, epoch, p.ar_budget_ns)) {
        atomicExch(p.status, ERR_WAIT_PEER);
        break;
      }
    }
  }

  // Common exit: every thread arrives here, then the allocating warp frees TMEM.
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // Give copies that may still be in flight time to land before smem is released.
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (p.ar_mode && threadIdx.x == 0) {
    // the last CTA to leave publishes the new epoch (every CTA read the old one before the first barrier)
    __threadfence();
    const uint32_t done = atomicAdd(&p.comm.ctrl[1], 1u) + 1;
    if (done == gridDim.x) {
      p.comm.ctrl[1] = 0;
      __threadfence();
      atomicExch(&p.comm.ctrl[0], ar_epoch_at_entry);
    }
  }
}

// Sum split-K partials (+ optional residual) into bf16.
static __global__ void splitk_reduce_kernel(const float* __restrict__ part, int splits, size_t n,
                                     const __nv_bfloat16* __restrict__ residual,
                                     __nv_bfloat16* __restrict__ out) {
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = residual ? __bfloat162float(residual[i]) : 0.f;
  for (int s = 0; s < splits; ++s) acc += part[(size_t)s * n + i];
  out[i] = __float2bfloat16(acc);
}

template <int BN, int WFMT>
static int launch_one(const CUtensorMap& tmW, const CUtensorMap& tmX, const GemmParams& p,
                      cudaStream_t stream) {
  using L = SmemLayout<BN, WFMT>;
  static b200::PerDeviceOnce once_;
  bool& configured = once_.slot();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_wdec_kernel<BN, WFMT>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  if (p.ar_mode == 3 && L::EPI_BYTES == 0) return -ERR_BAD_ARG;   // this instance has no epilogue staging
  const int total = p.work_table ? sm_count() : p.m_tiles * p.n_tiles * p.splits;
  const int grid = total < sm_count() ? total : sm_count();
  gemm_wdec_kernel<BN, WFMT><<<grid, NUM_THREADS, L::TOTAL, stream>>>(tmW, tmX, p);
  return (int)cudaGetLastError();
}

}  // namespace b200
