// Lightning indexer on the tensor cores: score[t, s] = scale * sum_h w[t, h] relu(q[t, h, :] . k[s, :]) for s <= pos[t].
// Per head the scores of a tile are a [queries x DI] x [DI x keys] product, so a CTA takes 128 queries x 64 keys: the
// key tile is gathered once from the paged index cache, the queries of one head at a time are streamed through a
// double-buffered shared-memory tile with cp.async, each of the 8 warps multiplies its 16 queries against the 64 keys
// (m16n8k16, bf16 operands through ldmatrix) and folds relu(.) times the head weight into fp32 totals in registers.
// Key tiles that lie entirely behind the causal frontier of the query tile are filled with -inf without any math.
//
// Same contract as the scalar kernel in attn_mla.cu (one thread per key, fp32 FMAs), which stays for batches that mix
// sequences (every query then has its own block table) and for index widths other than 64 / 128.
// Reference behaviour: the DeepSeek sparse-attention indexer scoring (src/models/deepseek_v4/runtime.py:1112-1288).
#include <cuda_bf16.h>
#include "per_device.h"
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int QT = 128;   // queries per CTA (16 per warp)
constexpr int KT = 64;    // keys per CTA

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

// grid (ceil(ld / 64), ceil(T / 128)), 256 threads.
template <int DI>
__global__ void __launch_bounds__(256, 2)
mla_indexer_mma_kernel(const __nv_bfloat16* __restrict__ q_idx, const float* __restrict__ hw,
                       const __nv_bfloat16* __restrict__ idx_cache, const int* __restrict__ block_table, int max_blocks, int bs,
                       const int* __restrict__ positions, float* __restrict__ scores, int ld, int T, int HI, float scale) {
  constexpr int LD = DI + 8;                                  // padded row (elements): ldmatrix rows fall in distinct banks
  extern __shared__ __align__(16) uint8_t smem[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem);            // [KT][LD]
  __nv_bfloat16* sQ = sK + KT * LD;                                      // [2][QT][LD]
  __shared__ int s_maxpos;
  const int k0 = blockIdx.x * KT, q0 = blockIdx.y * QT;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;

  if (tid == 0) s_maxpos = -1;
  __syncthreads();
  if (tid < QT && q0 + tid < T) atomicMax(&s_maxpos, positions[q0 + tid]);
  __syncthreads();
  const int maxpos = s_maxpos;
  if (k0 > maxpos) {                                          // behind the causal frontier of every query of the tile
    for (int i = tid; i < QT * KT; i += 256) {
      const int r = i / KT, c = i % KT;
      if (q0 + r < T && k0 + c < ld) scores[(size_t)(q0 + r) * ld + k0 + c] = -INFINITY;
    }
    return;
  }

  // key tile: four threads per key row
  {
    const int j = tid >> 2, part = tid & 3;
    const int kp = k0 + j;
    __nv_bfloat16* drow = sK + j * LD;
    if (kp <= maxpos && kp / bs < max_blocks) {
      const __nv_bfloat16* srow = idx_cache + ((size_t)block_table[kp / bs] * bs + kp % bs) * DI;
#pragma unroll
      for (int c = part; c < DI / 8; c += 4) cp16(drow + c * 8, srow + c * 8);
    } else {
#pragma unroll
      for (int c = part; c < DI / 8; c += 4) *reinterpret_cast<uint4*>(drow + c * 8) = make_uint4(0, 0, 0, 0);
    }
  }
  auto fetch_q = [&](int h) {                                 // queries of head h: two threads per query row
    __nv_bfloat16* dst = sQ + (size_t)(h & 1) * QT * LD;
    const int r = tid >> 1, part = tid & 1;
    __nv_bfloat16* drow = dst + r * LD;
    if (q0 + r < T) {
      const __nv_bfloat16* srow = q_idx + ((size_t)(q0 + r) * HI + h) * DI;
#pragma unroll
      for (int c = part; c < DI / 8; c += 2) cp16(drow + c * 8, srow + c * 8);
    } else {
#pragma unroll
      for (int c = part; c < DI / 8; c += 2) *reinterpret_cast<uint4*>(drow + c * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  fetch_q(0);                                                 // the key tile's copies ride in the same group

  float total[8][4];
#pragma unroll
  for (int n = 0; n < 8; ++n) total[n][0] = total[n][1] = total[n][2] = total[n][3] = 0.f;
  const int r0 = q0 + 16 * warp + g, r1 = r0 + 8;
  const float* w0p = hw + (size_t)min(r0, T - 1) * HI;
  const float* w1p = hw + (size_t)min(r1, T - 1) * HI;

  for (int h = 0; h < HI; ++h) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                          // head h landed; every warp is done with head h - 1
    if (h + 1 < HI) fetch_q(h + 1);
    const __nv_bfloat16* qt = sQ + (size_t)(h & 1) * QT * LD;
    float acc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
    const __nv_bfloat16* ap = qt + (16 * warp + (lane & 15)) * LD + (lane >> 4) * 8;
    // B through ldmatrix.x4: (keys n..n+7, k 0-7), (same keys, k 8-15), (keys n+8..n+15, k 0-7), (those, k 8-15)
    const __nv_bfloat16* bp = sK + ((lane & 7) + ((lane >> 4) & 1) * 8) * LD + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < DI / 16; ++ks) {
      uint32_t a[4];
      ldmatrix_x4(a, ap + ks * 16);
#pragma unroll
      for (int np = 0; np < 4; ++np) {
        uint32_t b[4];
        ldmatrix_x4(b, bp + (size_t)np * 16 * LD + ks * 16);
        mma_bf16(acc[2 * np], a, b[0], b[1]);
        mma_bf16(acc[2 * np + 1], a, b[2], b[3]);
      }
    }
    const float w0 = w0p[h], w1 = w1p[h];
#pragma unroll
    for (int n = 0; n < 8; ++n) {
      total[n][0] += w0 * fmaxf(acc[n][0], 0.f); total[n][1] += w0 * fmaxf(acc[n][1], 0.f);
      total[n][2] += w1 * fmaxf(acc[n][2], 0.f); total[n][3] += w1 * fmaxf(acc[n][3], 0.f);
    }
  }

#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int t = hf ? r1 : r0;
    if (t >= T) continue;
    const int pos = positions[t];
    float* row = scores + (size_t)t * ld;
#pragma unroll
    for (int n = 0; n < 8; ++n)
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int s = k0 + 8 * n + 2 * tig + e;
        if (s < ld) row[s] = s <= pos ? total[n][2 * hf + e] * scale : -INFINITY;
      }
  }
}

template <int DI>
int launch(const __nv_bfloat16* q, const float* hw, const __nv_bfloat16* kc, const int* bt, int max_blocks, int bs,
           const int* positions, float* scores, int ld, int T, int HI, float scale, cudaStream_t stream) {
  constexpr int SMEM = (KT + 2 * QT) * (DI + 8) * 2;
  static b200::PerDeviceOnce once_;
  bool& configured = once_.slot();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_indexer_mma_kernel<DI>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  mla_indexer_mma_kernel<DI><<<dim3((ld + KT - 1) / KT, (T + QT - 1) / QT), 256, SMEM, stream>>>(
      q, hw, kc, bt, max_blocks, bs, positions, scores, ld, T, HI, scale);
  return (int)cudaGetLastError();
}

}  // namespace

// One sequence (a single block-table row); q_idx [T, HI, DI] bf16, hw [T, HI] fp32, idx_cache [rows, DI] bf16,
// scores fp32 [T, ld].  DI 64 or 128.
extern "C" int b200_mla_indexer_mma(const void* q_idx, const float* hw, const void* idx_cache, const int* block_table,
                                    int max_blocks, int bs, const int* positions, float* scores, int ld, int T, int HI, int DI,
                                    float scale, cudaStream_t stream) {
  if (T <= 0 || ld <= 0 || HI <= 0 || bs <= 0) return -6;
  auto q = reinterpret_cast<const __nv_bfloat16*>(q_idx);
  auto kc = reinterpret_cast<const __nv_bfloat16*>(idx_cache);
  if (DI == 128) return launch<128>(q, hw, kc, block_table, max_blocks, bs, positions, scores, ld, T, HI, scale, stream);
  if (DI == 64) return launch<64>(q, hw, kc, block_table, max_blocks, bs, positions, scores, ld, T, HI, scale, stream);
  return -6;
}
