// Causal GQA flash-attention prefill over a paged KV cache, head_dim 128, sm_100a.
//
// One CTA = one 128-row query tile of one query head.  Warp roles:
//   warp 4  : TMA producer - Q once, then K and V tiles of 128 keys gathered
//             block by block through the sequence's block table (two-stage rings);
//   warp 5  : tcgen05.mma issuer - S = Q K^T into one of two TMEM S buffers
//             (S(j+1) is issued before P(j) V(j) so it overlaps the softmax),
//             then O += P V with P read from shared memory and V consumed
//             MN-major straight from its token-major TMA tile;
//   warps 0-3: softmax - one query row per thread (TMEM lane == row), online
//             max/sum in the exp2 domain, P written as bf16 into the swizzled
//             K-major A-operand layout; O lives in TMEM and is rescaled lazily,
//             only when a row max grows by more than 2^8.
// Epilogue: O / l, optional sigmoid output gate (Qwen "attn_output_gate"), bf16 store.
// All mbarrier waits are bounded and unwind through the common exit.
//
// Reference behaviour: cpp_engine/backends/cuda/kernels/qwen_gqa_optimized.cu
// (gqa_prefill_* kernels :326-1482, online softmax, causal mask) and the paged
// KV layout of cpp_engine/include/block_table.hpp:22-71.
#include <cuda_bf16.h>
#include "per_device.h"
#include "../ptx/sm100.cuh"
#include "tma_host.h"
#include "ops.h"

namespace b200 {
namespace attn {

constexpr int D = 128;          // head dim
constexpr int BQ = 128;         // query rows per CTA
constexpr int BKV = 128;        // keys per tile
constexpr int ATOM = 16384;     // bytes of one [128 x 64] bf16 swizzled atom
constexpr int TILE = 2 * ATOM;  // [128 x 128] bf16
constexpr int NTHREADS = 192;
constexpr int SMEM_BYTES = 6 * TILE + 1024 + 256;  // Q, K x2, V x2, P

struct Params {
  const int* block_table;  // [B, max_blocks]
  const int* q_start;      // [B] first row of the sequence inside Q / O
  const int* q_len;        // [B]
  const int* kv_len;       // [B] context length including the new tokens
  int max_blocks;
  int block_size;          // tokens per KV block (16, 32, 64 or 128)
  int n_q_heads, n_kv_heads;
  float scale_log2;        // softmax scale * log2(e)
  __nv_bfloat16* out;      // [T, Hq, D]
  const __nv_bfloat16* gate;  // optional [T, Hq, D], out *= sigmoid(gate)
  int* status;
  int window, sinks;       // window > 0: a query at position p sees keys (p - window, p] and the first `sinks` keys
};

__device__ __forceinline__ uint64_t desc_k_sw128(const void* p) { return umma_desc_sw128(p); }
// MN-major operand, 128B swizzle: 64-element MN atoms LBO bytes apart, 8-row K groups SBO bytes apart.
__device__ __forceinline__ uint64_t desc_mn_sw128(const void* p, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_u32(p) & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128);
constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 128) | (1u << 16);  // B is MN-major

__global__ void __launch_bounds__(NTHREADS, 1)
gqa_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                   const __grid_constant__ CUtensorMap tmV, Params p) {
  extern __shared__ uint8_t smem_base[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_base) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + TILE;      // 2 stages
  uint8_t* sV = sK + 2 * TILE;  // 2 stages
  uint8_t* sP = sV + 2 * TILE;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + TILE);
  uint64_t* q_full = bars;          // 1
  uint64_t* k_full = bars + 1;      // 2
  uint64_t* k_empty = bars + 3;     // 2
  uint64_t* v_full = bars + 5;      // 2
  uint64_t* v_empty = bars + 7;     // 2
  uint64_t* s_full = bars + 9;      // 2
  uint64_t* p_full = bars + 11;     // 1
  uint64_t* pv_done = bars + 12;    // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.z, h = blockIdx.y, qt = blockIdx.x;
  const int q_len = p.q_len[b];
  const int kv_len = p.kv_len[b];
  const int q0 = qt * BQ;
  if (q0 >= q_len) return;  // uniform per CTA, before any barrier/TMEM use
  const int q_row0 = p.q_start[b] + q0;
  const int kvh = h / (p.n_q_heads / p.n_kv_heads);
  const int pos0 = kv_len - q_len + q0;  // context position of the tile's first query row
  // Key tiles this query tile visits.  With a sliding window the tiles wholly below every row's window are
  // skipped, except the leading tiles that hold attention-sink keys: iteration j maps to tile_of(j).
  const int n_tiles_all = (min(kv_len, pos0 + BQ) + BKV - 1) / BKV;
  int n_sink_tiles = 0, first_win_tile = 0;
  if (p.window > 0) {
    first_win_tile = max(0, pos0 - p.window + 1) / BKV;
    n_sink_tiles = min(first_win_tile, (p.sinks + BKV - 1) / BKV);
  }
  const int n_tiles = n_sink_tiles + (n_tiles_all - first_win_tile);
  auto tile_of = [&](int j) { return j < n_sink_tiles ? j : first_win_tile + (j - n_sink_tiles); };

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(p_full, 128);
    mbar_init(pv_done, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // V stages start finite: rows of keys past the context are never loaded but still multiply P = 0.
  for (int i = threadIdx.x; i < 2 * TILE / 16; i += NTHREADS) reinterpret_cast<uint4*>(sV)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  const uint32_t tS[2] = {tmem, tmem + 128};
  const uint32_t tO = tmem + 256;

  if (warp == 4) {
    if (lane == 0) {
      tma_prefetch_desc(&tmQ);
      tma_prefetch_desc(&tmK);
      tma_prefetch_desc(&tmV);
      mbar_expect_tx(q_full, TILE);
      tma_load_2d(sQ, &tmQ, q_full, h * D, q_row0);
      tma_load_2d(sQ + ATOM, &tmQ, q_full, h * D + 64, q_row0);
      const int* bt = p.block_table + (size_t)b * p.max_blocks;
      const int bs = p.block_size;
      const int per_tile = BKV / bs;
      const uint32_t sub_bytes = bs * 128;  // one d-half of one block
      for (int j = 0; j < n_tiles && !*abort_flag; ++j) {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int key0 = tile_of(j) * BKV;
        int nblk = 0;
        for (int s = 0; s < per_tile; ++s)
          if (key0 + s * bs < kv_len) ++nblk;
        // K tile
        if (!mbar_wait(&k_empty[st], ph ^ 1)) { atomicExch(p.status, ERR_WAIT_STAGE); *abort_flag = 1; break; }
        mbar_expect_tx(&k_full[st], nblk * 2 * sub_bytes);
        for (int s = 0; s < nblk; ++s) {
          const int blk = bt[(key0 + s * bs) / bs];
          const int row = (blk * p.n_kv_heads + kvh) * bs;
          tma_load_2d(sK + st * TILE + s * sub_bytes, &tmK, &k_full[st], 0, row);
          tma_load_2d(sK + st * TILE + ATOM + s * sub_bytes, &tmK, &k_full[st], 64, row);
        }
        // V tile
        if (!mbar_wait(&v_empty[st], ph ^ 1)) { atomicExch(p.status, ERR_WAIT_STAGE); *abort_flag = 1; break; }
        mbar_expect_tx(&v_full[st], nblk * 2 * sub_bytes);
        for (int s = 0; s < nblk; ++s) {
          const int blk = bt[(key0 + s * bs) / bs];
          const int row = (blk * p.n_kv_heads + kvh) * bs;
          tma_load_2d(sV + st * TILE + s * sub_bytes, &tmV, &v_full[st], 0, row);
          tma_load_2d(sV + st * TILE + ATOM + s * sub_bytes, &tmV, &v_full[st], 64, row);
        }
      }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      bool ok = mbar_wait(q_full, 0);
      if (!ok) { atomicExch(p.status, ERR_WAIT_TMA); *abort_flag = 1; }
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
        tc_fence_after();
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16_ss(tS[st], desc_k_sw128(sQ + a * ATOM) + 2 * k, desc_k_sw128(sK + st * TILE + a * ATOM) + 2 * k,
                         idesc_qk, (a | k) ? 1u : 0u);
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      if (ok && n_tiles > 0) ok = issue_s(0);
      for (int j = 0; ok && j < n_tiles && !*abort_flag; ++j) {
        const int st = j & 1;
        if (j + 1 < n_tiles) {
          ok = issue_s(j + 1);
          if (!ok) break;
        }
        if (!mbar_wait(p_full, j & 1) || !mbar_wait(&v_full[st], (j >> 1) & 1)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint64_t da = desc_k_sw128(sP + (kk >> 2) * ATOM) + 2 * (kk & 3);
          const uint64_t db = desc_mn_sw128(sV + st * TILE + kk * 2048, ATOM, 1024);
          umma_bf16_ss(tO, da, db, idesc_pv, (j | kk) ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(pv_done);
      }
      if (!ok) { atomicExch(p.status, ERR_WAIT_TMA); *abort_flag = 1; }
    }
  } else {
    // ------------------------------------------------------------- softmax warps
    const int r = warp * 32 + lane;           // query row in the tile == TMEM lane
    const int limit = pos0 + r;               // last visible key index for this row
    const uint32_t lane_off = uint32_t(warp * 32) << 16;
    float m_run = -INFINITY, l_run = 0.f;
    bool alive = true;
    for (int j = 0; j < n_tiles; ++j) {
      const int sb = j & 1;
      bool ok = mbar_wait(&s_full[sb], (j >> 1) & 1);
      ok = __all_sync(0xffffffffu, ok) && !*abort_flag;
      if (!ok) { alive = false; break; }
      tc_fence_after();
      float s[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(tS[sb] + lane_off + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(v[i]) * p.scale_log2;
      }
      const int key0 = tile_of(j) * BKV;
      const int kmax = min(limit, kv_len - 1) - key0;  // keys with index > kmax are masked
      const int klo = p.window > 0 ? limit - p.window + 1 - key0 : -(1 << 30);   // keys below klo are outside the window
      float m_tile = -INFINITY;
      if (klo > 0) {
        const int ks = p.sinks - key0;                 // keys below ks are sinks and stay visible
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (i > kmax || (i < klo && i >= ks)) s[i] = -INFINITY;
          m_tile = fmaxf(m_tile, s[i]);
        }
      } else if (kmax < 127) {
#pragma unroll
        for (int i = 0; i < 128; ++i) {
          if (i > kmax) s[i] = -INFINITY;
          m_tile = fmaxf(m_tile, s[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 128; ++i) m_tile = fmaxf(m_tile, s[i]);
      }
      // P(j) overwrites the buffer P(j-1) V(j-1) reads, and O may be rescaled: wait for that MMA.
      if (j > 0) {
        bool ok2 = mbar_wait(pv_done, (j - 1) & 1);
        ok2 = __all_sync(0xffffffffu, ok2);
        if (!ok2) { alive = false; break; }
        tc_fence_after();
      }
      const float m_new = fmaxf(m_run, m_tile);
      const bool grow = m_new > m_run + 8.f;  // also true on the first tile (m_run = -inf) unless all masked
      if (j == 0) {
        m_run = (m_new == -INFINITY) ? 0.f : m_new;
      } else if (__any_sync(0xffffffffu, grow)) {
        const float m_next = grow ? m_new : m_run;
        const float alpha = (m_run == -INFINITY) ? 0.f : exp2f(m_run - m_next);
        l_run *= alpha;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + lane_off + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tO + lane_off + c * 32, v);
        }
        tmem_st_wait();
        m_run = m_next;
      }
      float lsum = 0.f;
      uint8_t* prow = sP + (r >> 3) * 1024 + (r & 7) * 128;
      const int sw = r & 7;
#pragma unroll
      for (int c8 = 0; c8 < 16; ++c8) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2f(s[c8 * 8 + i] - m_run);
          lsum += e[i];
        }
        uint4 u;
        __nv_bfloat162 t0 = __floats2bfloat162_rn(e[0], e[1]);
        __nv_bfloat162 t1 = __floats2bfloat162_rn(e[2], e[3]);
        __nv_bfloat162 t2 = __floats2bfloat162_rn(e[4], e[5]);
        __nv_bfloat162 t3 = __floats2bfloat162_rn(e[6], e[7]);
        u.x = *reinterpret_cast<uint32_t*>(&t0);
        u.y = *reinterpret_cast<uint32_t*>(&t1);
        u.z = *reinterpret_cast<uint32_t*>(&t2);
        u.w = *reinterpret_cast<uint32_t*>(&t3);
        *reinterpret_cast<uint4*>(prow + (c8 >> 3) * ATOM + (((c8 & 7) ^ sw) << 4)) = u;
      }
      l_run += lsum;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_full);
    }
    if (alive && n_tiles > 0) {
      bool ok = mbar_wait(pv_done, (n_tiles - 1) & 1);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        tc_fence_after();
        const float inv = l_run > 0.f ? 1.f / l_run : 0.f;
        const bool row_ok = (q0 + r) < q_len;
        const size_t orow = ((size_t)(q_row0 + r) * p.n_q_heads + h) * D;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(tO + lane_off + c * 32, v);
          tmem_ld_wait();
          if (row_ok) {
#pragma unroll
            for (int g8 = 0; g8 < 4; ++g8) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) o[i] = __uint_as_float(v[g8 * 8 + i]) * inv;
              if (p.gate) {
                const uint4 gu = *reinterpret_cast<const uint4*>(p.gate + orow + c * 32 + g8 * 8);
                const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gu);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 gf = __bfloat1622float2(gh[i]);
                  o[2 * i] *= 1.f / (1.f + __expf(-gf.x));
                  o[2 * i + 1] *= 1.f / (1.f + __expf(-gf.y));
                }
              }
              uint4 u;
              __nv_bfloat162 t0 = __floats2bfloat162_rn(o[0], o[1]);
              __nv_bfloat162 t1 = __floats2bfloat162_rn(o[2], o[3]);
              __nv_bfloat162 t2 = __floats2bfloat162_rn(o[4], o[5]);
              __nv_bfloat162 t3 = __floats2bfloat162_rn(o[6], o[7]);
              u.x = *reinterpret_cast<uint32_t*>(&t0);
              u.y = *reinterpret_cast<uint32_t*>(&t1);
              u.z = *reinterpret_cast<uint32_t*>(&t2);
              u.w = *reinterpret_cast<uint32_t*>(&t3);
              *reinterpret_cast<uint4*>(p.out + orow + c * 32 + g8 * 8) = u;
            }
          }
        }
      } else {
        alive = false;
      }
    }
    if (!alive) {
      if (lane == 0) atomicExch(p.status, ERR_WAIT_ACC);
      *abort_flag = 1;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    uint64_t t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace attn
}  // namespace b200

using namespace b200;

// q: [T, Hq, 128] bf16; k_cache / v_cache: [num_blocks, Hkv, block_size, 128] bf16 (zero-initialised
// at allocation); block_table: [B, max_blocks] int32; q_start/q_len/kv_len: [B] int32 (device).
// out: [T, Hq, 128] bf16; gate optional (same shape as out). max_q_len bounds the grid.
// Sliding-window setting of the next launch (set by b200_gqa_prefill_ex; 0 = full causal attention).
static thread_local int g_window = 0, g_sinks = 0;

extern "C" int b200_gqa_prefill(const void* q, const void* k_cache, const void* v_cache, void* out,
                                const void* gate, const int* block_table, const int* q_start,
                                const int* q_len, const int* kv_len, int batch, int max_q_len,
                                int total_q_rows, int max_blocks, int num_blocks, int block_size,
                                int n_q_heads, int n_kv_heads, float softmax_scale, int* status,
                                cudaStream_t stream) {
  using namespace b200::attn;
  if (block_size != 16 && block_size != 32 && block_size != 64 && block_size != 128) return -ERR_BAD_ARG;
  if (n_q_heads % n_kv_heads) return -ERR_BAD_ARG;
  static b200::PerDeviceOnce once_;
  bool& configured = once_.slot();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(gqa_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  CUtensorMap tmQ, tmK, tmV;
  bool ok = make_tmap_2d(&tmQ, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, q, total_q_rows, (uint64_t)n_q_heads * D,
                         (uint64_t)n_q_heads * D * 2, BQ, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  const uint64_t kv_rows = (uint64_t)num_blocks * n_kv_heads * block_size;
  ok = ok && make_tmap_2d(&tmK, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, k_cache, kv_rows, D, D * 2, block_size, 64,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  ok = ok && make_tmap_2d(&tmV, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v_cache, kv_rows, D, D * 2, block_size, 64,
                          CU_TENSOR_MAP_SWIZZLE_128B);
  if (!ok) return -ERR_BAD_ARG;
  Params p;
  p.block_table = block_table;
  p.q_start = q_start;
  p.q_len = q_len;
  p.kv_len = kv_len;
  p.max_blocks = max_blocks;
  p.block_size = block_size;
  p.n_q_heads = n_q_heads;
  p.n_kv_heads = n_kv_heads;
  p.scale_log2 = softmax_scale * 1.4426950408889634f;
  p.out = reinterpret_cast<__nv_bfloat16*>(out);
  p.gate = reinterpret_cast<const __nv_bfloat16*>(gate);
  p.status = status;
  p.window = g_window;
  p.sinks = g_sinks;
  dim3 grid((max_q_len + BQ - 1) / BQ, n_q_heads, batch);
  gqa_prefill_kernel<<<grid, NTHREADS, SMEM_BYTES, stream>>>(tmQ, tmK, tmV, p);
  return (int)cudaGetLastError();
}

// As b200_gqa_prefill, restricted to a sliding window with attention sinks: a query at position p attends to the keys
// (p - window, p] and to the first `sinks` keys of its sequence (window <= 0: full causal attention).
extern "C" int b200_gqa_prefill_ex(const void* q, const void* k_cache, const void* v_cache, void* out, const void* gate,
                                   const int* block_table, const int* q_start, const int* q_len, const int* kv_len, int batch,
                                   int max_q_len, int total_q_rows, int max_blocks, int num_blocks, int block_size,
                                   int n_q_heads, int n_kv_heads, float softmax_scale, int window, int sinks, int* status,
                                   cudaStream_t stream) {
  g_window = window > 0 ? window : 0;
  g_sinks = sinks > 0 ? sinks : 0;
  const int rc = b200_gqa_prefill(q, k_cache, v_cache, out, gate, block_table, q_start, q_len, kv_len, batch, max_q_len,
                                  total_q_rows, max_blocks, num_blocks, block_size, n_q_heads, n_kv_heads, softmax_scale, status,
                                  stream);
  g_window = g_sinks = 0;
  return rc;
}
