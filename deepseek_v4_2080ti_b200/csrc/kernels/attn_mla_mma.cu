// Absorbed multi-head latent attention on the tensor cores.
//
// All heads of a token attend to the same latent rows (one shared KV "head" of C latent + R rope dims), so for one
// query token the scores of up to 16 heads over a tile of keys are a [16 x (C+R)] x [(C+R) x keys] product and the
// output a [16 x keys] x [keys x C] product: the heads are the M dimension of m16n8k16 MMAs.  One CTA handles one
// token and one group of 16 heads: it gathers the token's selected cache rows (top-k indices of the sparse indexer, or
// the causal prefix) tile by tile with cp.async - once for all heads of the group, double-buffered - and keeps the
// running soft-max state and the [16 x C] output in registers.
//   warp w: scores of keys [8w, 8w+8) of each 32-key tile; output dims [w C/4, (w+1) C/4).
// The rows of a tile serve as the B operand twice: K-major for the scores, and through ldmatrix.trans as V.
//
// Reference behaviour: GLM MLA with absorbed k_b / v_b (src/models/glm_dsa/architecture.py:263-406) and the
// DeepSeek sparse attention dispatcher (src/kernels/ops.py:982-1100), which run per-head SDPA / Triton kernels.
#include <cuda_bf16.h>
#include "per_device.h"
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int KT = 32;        // keys per tile (= threads / 4: the gather assigns four threads to a key row)

__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ size_t cache_row_of(const int* bt, int bs, int pos) { return (size_t)bt[pos / bs] * bs + pos % bs; }

// MT: 16-head groups (m-tiles) per CTA; the CTA has 4 MT warps and gathers a token's rows once for 16 MT heads.
template <int C, int R, int MT>
struct Layout {
  static constexpr int HG = 16 * MT;
  static constexpr int D = C + R;
  static constexpr int LD = D + 8;                           // padded row (elements): 16-byte aligned, bank-skewed
  static constexpr int Q_BYTES = HG * LD * 2;
  static constexpr int K_BYTES = KT * LD * 2;
  static constexpr int PLD = KT + 8;                          // padded row (elements) of the probability tile
  static constexpr int P_BYTES = HG * PLD * 2;
  static constexpr int STAT_BYTES = 2 * 4 * HG * 4;           // per-warp partial row maxima and row sums
  static constexpr int TOTAL = Q_BYTES + 2 * K_BYTES + P_BYTES + STAT_BYTES + 2 * KT * 4;
};

// grid (T, ceil(H / (16 MT))), 128 MT threads.  Warp w: head group mt = w / 4, key / output-dim quarter qd = w % 4.
template <int C, int R, int MT>
__global__ void __launch_bounds__(128 * MT)
mla_attention_mma_kernel(const __nv_bfloat16* __restrict__ q_lat, const __nv_bfloat16* __restrict__ q_pe,
                         const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int max_blocks, int bs,
                         const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ sel,
                         int nsel, __nv_bfloat16* __restrict__ o_lat, int T, int H, float scale, float* __restrict__ part,
                         int splits) {
  using L = Layout<C, R, MT>;
  constexpr int D = L::D, LD = L::LD, HG = L::HG, NTHR = 128 * MT;
  constexpr int NT = C / 4 / 8;                               // output n-tiles per warp
  extern __shared__ __align__(16) uint8_t smem[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem);
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem + L::Q_BYTES);
  __nv_bfloat16* sP = reinterpret_cast<__nv_bfloat16*>(smem + L::Q_BYTES + 2 * L::K_BYTES);   // [16][PLD] probabilities
  float* sMax = reinterpret_cast<float*>(smem + L::Q_BYTES + 2 * L::K_BYTES + L::P_BYTES);    // [4 warps][16 rows]
  float* sSum = sMax + 4 * HG;                                                                // [4 warps][16 rows]
  int* sPos = reinterpret_cast<int*>(sSum + 4 * HG);                           // [2][KT] key position, -1 = masked
  const int t = blockIdx.x, h0 = blockIdx.y * HG;
  const int tid = threadIdx.x, lane = tid & 31, g = lane >> 2, tig = lane & 3;
  const int warp = (tid >> 5) & 3, mt = tid >> 7;             // quarter and head group of this warp
  const int pos = positions[t];
  const int* bt = block_table + (size_t)(seq_of_token ? seq_of_token[t] : 0) * max_blocks;
  const int nkeys = sel ? nsel : pos + 1;
  const int ntiles_all = (nkeys + KT - 1) / KT;
  // split-KV (decode): CTA z takes a contiguous share of the tiles and leaves an unnormalised partial state
  const int per_split = (ntiles_all + splits - 1) / splits;
  const int tile_lo = blockIdx.z * per_split, ntiles = min(ntiles_all, tile_lo + per_split);

  // four threads per key row: the row's cache address (selection entry, block table, division by the block size) is
  // worked out once per thread and tile, then 18 copies of 16 bytes go out back to back
  auto fetch = [&](int tile) {
    __nv_bfloat16* dst = sK + (size_t)(tile & 1) * KT * LD;
    int* dpos = sPos + (tile & 1) * KT;
    constexpr int TPK = NTHR / KT;                            // threads per key row
    const int j = tid / TPK, part = tid % TPK;
    const int key = tile * KT + j;
    int kp = -1;
    if (key < nkeys) kp = sel ? sel[(size_t)t * nsel + key] : key;
    if (kp > pos) kp = -1;
    if (part == 0) dpos[j] = kp;
    __nv_bfloat16* drow = dst + j * LD;
    if (kp >= 0) {
      const __nv_bfloat16* srow = cache + cache_row_of(bt, bs, kp) * D;
#pragma unroll
      for (int c = part; c < D / 8; c += TPK) cp16(drow + c * 8, srow + c * 8);
    } else {
#pragma unroll
      for (int c = part; c < D / 8; c += TPK) *reinterpret_cast<uint4*>(drow + c * 8) = make_uint4(0, 0, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  // queries of this head group: rows = heads (rows past H stay zero)
  for (int i = tid; i < HG * (D / 8); i += NTHR) {
    const int r = i / (D / 8), c = i % (D / 8);
    uint4 u = make_uint4(0, 0, 0, 0);
    if (h0 + r < H) {
      if (c * 8 < C) u = *reinterpret_cast<const uint4*>(q_lat + ((size_t)(h0 + r) * T + t) * C + c * 8);
      else u = *reinterpret_cast<const uint4*>(q_pe + ((size_t)t * H + h0 + r) * R + (c * 8 - C));
    }
    *reinterpret_cast<uint4*>(sQ + r * LD + c * 8) = u;
  }
  if (tile_lo < ntiles) fetch(tile_lo);

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};   // rows g and g + 8

  for (int tile = tile_lo; tile < ntiles; ++tile) {
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();                                   // tile landed; previous tile's readers are done
    if (tile + 1 < ntiles) fetch(tile + 1);
    const __nv_bfloat16* kt = sK + (size_t)(tile & 1) * KT * LD;
    const int* kpos = sPos + (tile & 1) * KT;
    // ---- scores of keys [8 warp, 8 warp + 8): S[16 x 8] = Q[16 x D] K^T, operands through ldmatrix (two k-steps per
    // B load)
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    {
      const __nv_bfloat16* ap = sQ + (16 * mt + (lane & 15)) * LD + (lane >> 4) * 8;
      const __nv_bfloat16* bp = kt + (8 * warp + (lane & 7)) * LD + (lane >> 3) * 8;
#pragma unroll 6
      for (int ks = 0; ks < D / 16; ks += 2) {
        uint32_t a0[4], a1[4], b[4];
        ldmatrix_x4(a0, ap + ks * 16);
        ldmatrix_x4(a1, ap + ks * 16 + 16);
        ldmatrix_x4(b, bp + ks * 16);
        mma_bf16(s, a0, b[0], b[1]);
        mma_bf16(s, a1, b[2], b[3]);
      }
    }
    // ---- soft-max, computed once: every warp owns 8 keys of the tile; row statistics are exchanged through shared memory
    {
      const int kc = 8 * warp + 2 * tig;
      const bool v0 = kpos[kc] >= 0, v1 = kpos[kc + 1] >= 0;
      s[0] = v0 ? s[0] * scale : -INFINITY; s[1] = v1 ? s[1] * scale : -INFINITY;
      s[2] = v0 ? s[2] * scale : -INFINITY; s[3] = v1 ? s[3] * scale : -INFINITY;
      float mx0 = fmaxf(s[0], s[1]), mx1 = fmaxf(s[2], s[3]);
      mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
      mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
      if (tig == 0) { sMax[warp * HG + 16 * mt + g] = mx0; sMax[warp * HG + 16 * mt + g + 8] = mx1; }
    }
    __syncthreads();
    float corr[2];
    {
      float mx[2];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        const int r = 16 * mt + g + 8 * hf;
        mx[hf] = fmaxf(fmaxf(m_run[hf], fmaxf(sMax[r], sMax[HG + r])), fmaxf(sMax[2 * HG + r], sMax[3 * HG + r]));
        corr[hf] = (m_run[hf] == -INFINITY) ? 0.f : __expf(m_run[hf] - mx[hf]);
        m_run[hf] = mx[hf];
      }
      const float e0 = mx[0] == -INFINITY ? 0.f : __expf(s[0] - mx[0]), e1 = mx[0] == -INFINITY ? 0.f : __expf(s[1] - mx[0]);
      const float e2 = mx[1] == -INFINITY ? 0.f : __expf(s[2] - mx[1]), e3 = mx[1] == -INFINITY ? 0.f : __expf(s[3] - mx[1]);
      const int kc = 8 * warp + 2 * tig;
      *reinterpret_cast<uint32_t*>(sP + (16 * mt + g) * L::PLD + kc) = pack_bf16(e0, e1);
      *reinterpret_cast<uint32_t*>(sP + (16 * mt + g + 8) * L::PLD + kc) = pack_bf16(e2, e3);
      float sm0 = e0 + e1, sm1 = e2 + e3;
      sm0 += __shfl_xor_sync(0xffffffffu, sm0, 1); sm0 += __shfl_xor_sync(0xffffffffu, sm0, 2);
      sm1 += __shfl_xor_sync(0xffffffffu, sm1, 1); sm1 += __shfl_xor_sync(0xffffffffu, sm1, 2);
      if (tig == 0) { sSum[warp * HG + 16 * mt + g] = sm0; sSum[warp * HG + 16 * mt + g + 8] = sm1; }
    }
    __syncthreads();
    uint32_t pa[2][4];                                 // P as the A operand of two k-steps (16 keys each)
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const int r = 16 * mt + g + 8 * hf;
      l_run[hf] = l_run[hf] * corr[hf] + (sSum[r] + sSum[HG + r]) + (sSum[2 * HG + r] + sSum[3 * HG + r]);
    }
    ldmatrix_x4(pa[0], sP + (16 * mt + (lane & 15)) * L::PLD + (lane >> 4) * 8);
    ldmatrix_x4(pa[1], sP + (16 * mt + (lane & 15)) * L::PLD + 16 + (lane >> 4) * 8);
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= corr[0]; o[n][1] *= corr[0];
      o[n][2] *= corr[1]; o[n][3] *= corr[1];
    }
    // ---- O[16 x C/4] += P[16 x 32] V[32 x C/4]; V = the latent part of the same rows, read transposed
#pragma unroll
    for (int ks = 0; ks < 2; ++ks) {
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        // x4: (keys 0-7, dims n), (keys 8-15, dims n), (keys 0-7, dims n+1), (keys 8-15, dims n+1)
        const int key = 16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int dim = warp * (C / 4) + (n + (lane >> 4)) * 8;
        uint32_t b[4];
        ldmatrix_x4_trans(b, kt + key * LD + dim);
        mma_bf16(o[n], pa[ks], b[0], b[1]);
        mma_bf16(o[n + 1], pa[ks], b[2], b[3]);
      }
    }
  }
  // ---- normalise and store (or leave the partial state of this split): rows = heads g, g + 8
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    const int h = h0 + 16 * mt + g + 8 * hf;
    if (h >= H) continue;
    if (part) {
      float* dst = part + (((size_t)t * H + h) * splits + blockIdx.z) * (C + 2);
#pragma unroll
      for (int n = 0; n < NT; ++n)
        *reinterpret_cast<float2*>(dst + warp * (C / 4) + 8 * n + 2 * tig) = make_float2(o[n][2 * hf], o[n][2 * hf + 1]);
      if (warp == 0 && tig == 0) { dst[C] = m_run[hf]; dst[C + 1] = l_run[hf]; }
      continue;
    }
    const float inv = l_run[hf] > 0.f ? 1.f / l_run[hf] : 0.f;
    __nv_bfloat16* dst = o_lat + ((size_t)h * T + t) * C + warp * (C / 4) + 2 * tig;
#pragma unroll
    for (int n = 0; n < NT; ++n)
      *reinterpret_cast<uint32_t*>(dst + 8 * n) = pack_bf16(o[n][2 * hf] * inv, o[n][2 * hf + 1] * inv);
  }
}

// grid T * H, 128 threads: combine the splits' (max, sum, unnormalised output) states (splits <= 32).
template <int C>
__global__ void mla_attention_merge_kernel(const float* __restrict__ part, int splits, __nv_bfloat16* __restrict__ o_lat, int T, int H) {
  __shared__ float wgt[32];
  __shared__ float s_inv;
  const int t = blockIdx.x / H, h = blockIdx.x % H;
  const float* base = part + (size_t)blockIdx.x * splits * (C + 2);
  if (threadIdx.x < 32) {
    const int s = threadIdx.x;
    const float m = s < splits ? base[(size_t)s * (C + 2) + C] : -INFINITY;
    const float l = s < splits ? base[(size_t)s * (C + 2) + C + 1] : 0.f;
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    const float w = m == -INFINITY ? 0.f : __expf(m - M);
    float Lsum = l * w;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) Lsum += __shfl_xor_sync(0xffffffffu, Lsum, o);
    wgt[s] = w;
    if (s == 0) s_inv = Lsum > 0.f ? 1.f / Lsum : 0.f;
  }
  __syncthreads();
  const float inv = s_inv;
  for (int d = threadIdx.x; d < C; d += blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < splits; ++s) acc += base[(size_t)s * (C + 2) + d] * wgt[s];
    o_lat[((size_t)h * T + t) * C + d] = __float2bfloat16(acc * inv);
  }
}

template <int C, int R, int MT>
int launch_mt(const __nv_bfloat16* ql, const __nv_bfloat16* qp, const __nv_bfloat16* kc, const int* block_table, int max_blocks,
              int bs, const int* positions, const int* seq_of_token, const int* sel, int nsel, __nv_bfloat16* ol, int T, int H,
              float scale, float* part, int splits, cudaStream_t stream) {
  using L = Layout<C, R, MT>;
  static b200::PerDeviceOnce once_;
  bool& configured = once_.slot();
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(mla_attention_mma_kernel<C, R, MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  mla_attention_mma_kernel<C, R, MT><<<dim3(T, (H + L::HG - 1) / L::HG, splits), 128 * MT, L::TOTAL, stream>>>(
      ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, ol, T, H, scale, splits > 1 ? part : nullptr,
      splits);
  if (splits > 1) mla_attention_merge_kernel<C><<<T * H, 128, 0, stream>>>(part, splits, ol, T, H);
  return (int)cudaGetLastError();
}

// Heads per CTA: as many as keep the grid at a wave or more (the gather of a token's rows is shared by the CTA's heads);
// with few tokens (decode) 16 heads per CTA and the context split over `splits` CTAs.
template <int C, int R>
int launch(const __nv_bfloat16* ql, const __nv_bfloat16* qp, const __nv_bfloat16* kc, const int* block_table, int max_blocks,
           int bs, const int* positions, const int* seq_of_token, const int* sel, int nsel, __nv_bfloat16* ol, int T, int H,
           float scale, float* part, int splits, cudaStream_t stream) {
  if (splits < 1 || splits > 32 || (splits > 1 && !part)) return -6;
  if (splits == 1 && H > 32 && (long long)T * ((H + 63) / 64) >= 148 && Layout<C, R, 4>::TOTAL <= 227 * 1024)
    return launch_mt<C, R, 4>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, ol, T, H, scale, part, 1, stream);
  if (splits == 1 && H > 16 && (long long)T * ((H + 31) / 32) >= 148)
    return launch_mt<C, R, 2>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, ol, T, H, scale, part, 1, stream);
  return launch_mt<C, R, 1>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, ol, T, H, scale, part, splits, stream);
}

}  // namespace

// Same contract as b200_mla_attention (attn_mla.cu): q_lat [H, T, C], q_pe [T, H, R], cache [rows, C + R] bf16,
// o_lat [H, T, C]; sel int32 [T, nsel] cache positions (-1 = unused) or null for the causal prefix.
// splits > 1 (decode): the context of every token is cut into `splits` shares handled by separate CTAs; workspace is
// fp32 [T * H * splits * (C + 2)].
extern "C" int b200_mla_attention_splitkv(const void* q_lat, const void* q_pe, const void* cache, const int* block_table,
                                          int max_blocks, int bs, const int* positions, const int* seq_of_token, const int* sel,
                                          int nsel, void* o_lat, int T, int H, int C, int R, float scale, float* workspace,
                                          int splits, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return -6;
  auto ql = reinterpret_cast<const __nv_bfloat16*>(q_lat);
  auto qp = reinterpret_cast<const __nv_bfloat16*>(q_pe);
  auto kc = reinterpret_cast<const __nv_bfloat16*>(cache);
  auto ol = reinterpret_cast<__nv_bfloat16*>(o_lat);
  if (C == 512 && R == 64)
    return launch<512, 64>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, ol, T, H, scale, workspace,
                           splits, stream);
  if (C == 128 && R == 32)
    return launch<128, 32>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, ol, T, H, scale, workspace,
                           splits, stream);
  // rows [value (128) | key (128)]: grouped-query attention over selected tokens (ops/qsa.py drives it with a zero
  // "latent" query, so the score is q . key and the output P . value)
  if (C == 128 && R == 128)
    return launch<128, 128>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, ol, T, H, scale, workspace,
                            splits, stream);
  return -6;
}

extern "C" int b200_mla_attention_mma(const void* q_lat, const void* q_pe, const void* cache, const int* block_table,
                                      int max_blocks, int bs, const int* positions, const int* seq_of_token, const int* sel,
                                      int nsel, void* o_lat, int T, int H, int C, int R, float scale, cudaStream_t stream) {
  return b200_mla_attention_splitkv(q_lat, q_pe, cache, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, o_lat, T,
                                    H, C, R, scale, nullptr, 1, stream);
}
