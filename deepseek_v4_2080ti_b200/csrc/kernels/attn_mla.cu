// Multi-head Latent Attention in the absorbed form, over a paged latent cache, with the sparse top-k indexer.
//   cache row (per token, shared by all heads): [kv_lora_rank normalised latent | rope_dim rotated key]  (bf16)
//   mla_kv_append   - RMSNorm of the latent part, interleaved RoPE of the key part, write to the token's cache row;
//                     the same launch normalises and stores the indexer key.
//   mla_q_prepare   - splits q [T, H, nope + rope]: nope part transposed to [H, T, nope] (operand of the per-head
//                     absorption GEMM q_nope W_uk), rope part rotated in place.
//   mla_indexer     - score[t, s] = sum_h w[t,h] relu(q_idx[t,h,:] . k_idx[s,:]) * scale for s <= pos[t]
//   topk_rows       - per-row top-k by radix select (values compared as ordered 32-bit keys)
//   mla_attention   - per (token, head): softmax over the selected (or all causal) cache rows of
//                     (q_lat . c + q_pe . k_pe) * scale, output sum_s p_s c_s  [kv_lora_rank]
//   transpose_heads - [H, T, D] -> [T, H, D]
// All of these are CUDA-core kernels: exact for decode (bounded by top-k keys per query) and for moderate prompts.
// Reference behaviour: MLA of the GLM runtime (src/models/glm_dsa/architecture.py:345-406), indexer of the DeepSeek-V4
// runtime (src/models/deepseek_v4/runtime.py:1112-1288), sparse attention kernels
// (cpp_engine/backends/cuda/kernels/cuda_ops.cu:951-1850, indexer :1857-1990).
#include <cuda_bf16.h>
#include <stdint.h>
#include "ops.h"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ size_t cache_row(const int* block_table, int bs, int pos) {
  return (size_t)block_table[pos / bs] * bs + pos % bs;
}

// grid T, block 256. kv [T, C + R] bf16; cache [rows, C + R]; slots [T] absolute cache rows (or < 0 to skip).
__global__ void mla_kv_append_kernel(const __nv_bfloat16* __restrict__ kv, const __nv_bfloat16* __restrict__ gamma, float eps,
                                     const int* __restrict__ positions, const int* __restrict__ slots, float theta,
                                     __nv_bfloat16* __restrict__ cache, int C, int R,
                                     const __nv_bfloat16* __restrict__ kidx, const __nv_bfloat16* __restrict__ kidx_gamma,
                                     __nv_bfloat16* __restrict__ idx_cache, int DI) {
  __shared__ float red[8];
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const __nv_bfloat16* row = kv + (size_t)t * (C + R);
  __nv_bfloat16* dst = cache + (size_t)slot * (C + R);
  float ss = 0.f;
  for (int i = threadIdx.x; i < C; i += blockDim.x) {
    const float v = __bfloat162float(row[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
  const float inv = rsqrtf(tot / (float)C + eps);
  for (int i = threadIdx.x; i < C; i += blockDim.x)
    dst[i] = __float2bfloat16(__bfloat162float(row[i]) * inv * __bfloat162float(gamma[i]));
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < R / 2; i += blockDim.x) {
    const float ang = pos * powf(theta, -2.f * (float)i / (float)R);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float a = __bfloat162float(row[C + 2 * i]), b = __bfloat162float(row[C + 2 * i + 1]);
    dst[C + 2 * i] = __float2bfloat16(a * cs - b * sn);
    dst[C + 2 * i + 1] = __float2bfloat16(a * sn + b * cs);
  }
  if (kidx) {
    __syncthreads();
    const __nv_bfloat16* kr = kidx + (size_t)t * DI;
    float s2 = 0.f;
    for (int i = threadIdx.x; i < DI; i += blockDim.x) {
      const float v = __bfloat162float(kr[i]);
      s2 += v * v;
    }
    s2 = warp_sum(s2);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s2;
    __syncthreads();
    float t2 = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t2 += red[w];
    const float inv2 = rsqrtf(t2 / (float)DI + eps);
    for (int i = threadIdx.x; i < DI; i += blockDim.x)
      idx_cache[(size_t)slot * DI + i] = __float2bfloat16(__bfloat162float(kr[i]) * inv2 * __bfloat162float(kidx_gamma[i]));
  }
}

// grid (T, H), block 64. q [T, H, N + R]: writes qn_t [H, T, N] and rotates the rope part into q_pe [T, H, R].
__global__ void mla_q_prepare_kernel(const __nv_bfloat16* __restrict__ q, const int* __restrict__ positions, float theta,
                                     __nv_bfloat16* __restrict__ qn_t, __nv_bfloat16* __restrict__ q_pe, int T, int H,
                                     int N, int R) {
  const int t = blockIdx.x, h = blockIdx.y;
  const __nv_bfloat16* src = q + ((size_t)t * H + h) * (N + R);
  for (int i = threadIdx.x; i < N; i += blockDim.x) qn_t[((size_t)h * T + t) * N + i] = src[i];
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < R / 2; i += blockDim.x) {
    const float ang = pos * powf(theta, -2.f * (float)i / (float)R);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    const float a = __bfloat162float(src[N + 2 * i]), b = __bfloat162float(src[N + 2 * i + 1]);
    q_pe[((size_t)t * H + h) * R + 2 * i] = __float2bfloat16(a * cs - b * sn);
    q_pe[((size_t)t * H + h) * R + 2 * i + 1] = __float2bfloat16(a * sn + b * cs);
  }
}

// grid (ceil(S/128), T), block 128: one thread per key. q_idx [T, HI, DI]; hw [T, HI] fp32 head weights (scaled);
// idx_cache [rows, DI]; scores [T, ld] fp32 (-inf beyond pos[t]).
template <int DI>
__global__ void __launch_bounds__(128)
mla_indexer_kernel(const __nv_bfloat16* __restrict__ q_idx, const float* __restrict__ hw,
                   const __nv_bfloat16* __restrict__ idx_cache, const int* __restrict__ block_table, int max_blocks,
                   int bs, const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                   float* __restrict__ scores, int ld, int HI, float scale) {
  extern __shared__ float sm[];      // [HI][DI] queries of this token, then [HI] weights
  const int t = blockIdx.y;
  const int s = blockIdx.x * 128 + threadIdx.x;
  const int pos = positions[t];
  if (blockIdx.x * 128 > pos) {
    if (s < ld) scores[(size_t)t * ld + s] = -INFINITY;
    return;
  }
  float* sq = sm;
  float* sw = sm + HI * DI;
  for (int i = threadIdx.x; i < HI * DI; i += 128) sq[i] = __bfloat162float(q_idx[(size_t)t * HI * DI + i]);
  for (int i = threadIdx.x; i < HI; i += 128) sw[i] = hw[(size_t)t * HI + i];
  __syncthreads();
  if (s >= ld) return;
  if (s > pos) {
    scores[(size_t)t * ld + s] = -INFINITY;
    return;
  }
  const int* bt = block_table + (size_t)(seq_of_token ? seq_of_token[t] : 0) * max_blocks;
  const __nv_bfloat16* kr = idx_cache + cache_row(bt, bs, s) * DI;
  float k[DI];
#pragma unroll
  for (int i = 0; i < DI; i += 8) {
    const uint4 u = *reinterpret_cast<const uint4*>(kr + i);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      k[i + 2 * e] = f.x;
      k[i + 2 * e + 1] = f.y;
    }
  }
  float acc = 0.f;
  for (int h = 0; h < HI; ++h) {
    const float* qh = sq + h * DI;
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < DI; ++i) d += qh[i] * k[i];
    acc += sw[h] * fmaxf(d, 0.f);
  }
  scores[(size_t)t * ld + s] = acc * scale;
}

__device__ __forceinline__ uint32_t ordered_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// One block (256 threads) per row: indices of the k largest values among the first n[row] entries.
// Output idx [rows, k], padded with -1 when fewer than k entries exist; order inside a row is unspecified.
__global__ void __launch_bounds__(1024)
topk_rows_kernel(const float* __restrict__ vals, int ld, const int* __restrict__ n_valid, int k, int* __restrict__ idx) {
  __shared__ int hist[256];
  __shared__ uint32_t s_prefix, s_mask;
  __shared__ int s_need, s_count_gt, s_count_eq;
  const int row = blockIdx.x;
  const int n = min(n_valid[row], ld);
  const float* v = vals + (size_t)row * ld;
  int* out = idx + (size_t)row * k;
  if (n <= k) {
    for (int i = threadIdx.x; i < k; i += blockDim.x) out[i] = i < n ? i : -1;
    return;
  }
  if (threadIdx.x == 0) { s_prefix = 0; s_mask = 0; s_need = k; }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int n_up = (n + blockDim.x - 1) / blockDim.x * blockDim.x;       // uniform trip count: ballots need whole warps
  // find the key of the k-th largest value, 8 bits at a time from the top.  Scores of one row share most of their
  // leading bits, so lanes that hit the same bin add to it once (match_any), not 32 times.
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (threadIdx.x < 256) hist[threadIdx.x] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix, mask = s_mask;
    for (int i = threadIdx.x; i < n_up; i += blockDim.x) {
      const uint32_t key = i < n ? ordered_key(v[i]) : 0u;
      const bool in = i < n && (key & mask) == prefix;
      const uint32_t act = __ballot_sync(0xffffffffu, in);
      if (in) {
        const int bin = (key >> shift) & 0xFF;
        const uint32_t peers = __match_any_sync(act, bin);
        if (lane == __ffs(peers) - 1) atomicAdd(&hist[bin], __popc(peers));
      }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int need = s_need, b = 255;
      for (; b > 0; --b) {
        if (hist[b] >= need) break;
        need -= hist[b];
      }
      s_need = need;
      s_prefix = prefix | ((uint32_t)b << shift);
      s_mask = mask | (0xFFu << shift);
    }
    __syncthreads();
  }
  const uint32_t kth = s_prefix;
  const int need_eq = s_need;          // how many entries equal to the k-th key are taken (lowest indices first)
  if (threadIdx.x == 0) { s_count_gt = 0; s_count_eq = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n_up; i += blockDim.x) {
    const bool gt = i < n && ordered_key(v[i]) > kth;
    const uint32_t m = __ballot_sync(0xffffffffu, gt);
    int base = 0;
    if (lane == 0 && m) base = atomicAdd(&s_count_gt, __popc(m));
    base = __shfl_sync(0xffffffffu, base, 0);
    if (gt) out[base + __popc(m & ((1u << lane) - 1))] = i;
  }
  __syncthreads();
  const int base = s_count_gt;
  // ties: deterministic choice of the lowest indices.  Every thread counts the ties of one contiguous segment, the
  // counts are scanned by thread 0, and a second pass writes the ties whose rank is below the number needed.
  {
    __shared__ int seg_base[1024];
    const int seg = (n + blockDim.x - 1) / blockDim.x;
    const int lo = min(n, (int)threadIdx.x * seg), hi = min(n, lo + seg);
    int c = 0;
    for (int i = lo; i < hi; ++i) c += ordered_key(v[i]) == kth;
    seg_base[threadIdx.x] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
      int run = 0;
      for (int w = 0; w < (int)blockDim.x; ++w) { const int x = seg_base[w]; seg_base[w] = run; run += x; }
    }
    __syncthreads();
    int r = seg_base[threadIdx.x];
    if (c > 0 && r < need_eq) {
      for (int i = lo; i < hi && r < need_eq; ++i)
        if (ordered_key(v[i]) == kth) out[base + r++] = i;
    }
  }
}

// grid (T, H), block 128 (4 warps).  Keys are visited in tiles of 32: lane j of every warp scores key j (warps split
// the latent dimension), then each thread owns C/128 output dims.  sel [T, nsel] cache positions (-1 = unused) or null
// for all positions 0..pos[t].
template <int C, int R>
__global__ void __launch_bounds__(128)
mla_attention_kernel(const __nv_bfloat16* __restrict__ q_lat, const __nv_bfloat16* __restrict__ q_pe,
                     const __nv_bfloat16* __restrict__ cache, const int* __restrict__ block_table, int max_blocks, int bs,
                     const int* __restrict__ positions, const int* __restrict__ seq_of_token, const int* __restrict__ sel,
                     int nsel, __nv_bfloat16* __restrict__ o_lat, int T, int H, float scale) {
  constexpr int D = C + R;
  constexpr int DP = D + 2;                 // padded row: stride of 289 words for D = 576 keeps the lanes on different banks
  constexpr int OPT = C / 128;              // output dims per thread
  __shared__ __nv_bfloat16 sk[32][DP];
  __shared__ float sq[D];
  __shared__ float part[4][32];
  __shared__ float sp[32];
  const int t = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pos = positions[t];
  const int* bt = block_table + (size_t)(seq_of_token ? seq_of_token[t] : 0) * max_blocks;
  const __nv_bfloat16* ql = q_lat + ((size_t)h * T + t) * C;
  const __nv_bfloat16* qp = q_pe + ((size_t)t * H + h) * R;
  for (int i = threadIdx.x; i < C; i += 128) sq[i] = __bfloat162float(ql[i]) * scale;
  for (int i = threadIdx.x; i < R; i += 128) sq[C + i] = __bfloat162float(qp[i]) * scale;
  const int nkeys = sel ? nsel : pos + 1;
  float m = -INFINITY, l = 0.f;
  float acc[OPT];
#pragma unroll
  for (int i = 0; i < OPT; ++i) acc[i] = 0.f;
  for (int k0 = 0; k0 < nkeys; k0 += 32) {
    __syncthreads();
    // gather 32 cache rows (16-byte pieces; D % 8 == 0)
    for (int i = threadIdx.x; i < 32 * (D / 8); i += 128) {
      const int j = i / (D / 8), c = i % (D / 8);
      int kp = -1;
      if (k0 + j < nkeys) kp = sel ? sel[(size_t)t * nsel + k0 + j] : k0 + j;
      uint4 u = make_uint4(0, 0, 0, 0);
      if (kp >= 0 && kp <= pos) u = *reinterpret_cast<const uint4*>(cache + cache_row(bt, bs, kp) * D + c * 8);
      // rows are padded by 2 elements, so 16-byte stores would be misaligned: store as four 32-bit words
      uint32_t* d32 = reinterpret_cast<uint32_t*>(&sk[j][c * 8]);
      d32[0] = u.x; d32[1] = u.y; d32[2] = u.z; d32[3] = u.w;
    }
    __syncthreads();
    // scores: warp w covers dims [w*D/4, (w+1)*D/4) of key `lane`
    {
      float d = 0.f;
      const int lo = warp * (D / 4), hi = lo + D / 4;
      for (int i = lo; i < hi; i += 2) {
        const float2 kf = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&sk[lane][i]));
        d += sq[i] * kf.x + sq[i + 1] * kf.y;
      }
      part[warp][lane] = d;
    }
    __syncthreads();
    int kp = -1;
    if (k0 + lane < nkeys) kp = sel ? sel[(size_t)t * nsel + k0 + lane] : k0 + lane;
    const bool valid = kp >= 0 && kp <= pos;
    const float s = valid ? part[0][lane] + part[1][lane] + part[2][lane] + part[3][lane] : -INFINITY;
    const float mt = fmaxf(m, warp_max(s));
    const float p = valid ? __expf(s - mt) : 0.f;
    const float corr = (m == -INFINITY) ? 0.f : __expf(m - mt);
    l = l * corr + warp_sum(p);
    m = mt;
    if (warp == 0) sp[lane] = p;
    __syncthreads();
#pragma unroll
    for (int i = 0; i < OPT; ++i) acc[i] *= corr;
    for (int j = 0; j < 32; ++j) {
      const float pj = sp[j];
      if (pj == 0.f) continue;
#pragma unroll
      for (int i = 0; i < OPT; ++i) acc[i] += pj * __bfloat162float(sk[j][threadIdx.x + 128 * i]);
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  __nv_bfloat16* o = o_lat + ((size_t)h * T + t) * C;
#pragma unroll
  for (int i = 0; i < OPT; ++i) o[threadIdx.x + 128 * i] = __float2bfloat16(acc[i] * inv);
}

// [H, T, D] -> [T, H, D]
__global__ void transpose_heads_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out, int H, int T, int D) {
  const int t = blockIdx.x, h = blockIdx.y;
  for (int i = threadIdx.x; i < D; i += blockDim.x) out[((size_t)t * H + h) * D + i] = in[((size_t)h * T + t) * D + i];
}

}  // namespace

extern "C" {

int b200_mla_kv_append(const void* kv, const void* gamma, float eps, const int* positions, const int* slots, float theta,
                       void* cache, int T, int C, int R, const void* kidx, const void* kidx_gamma, void* idx_cache, int DI,
                       cudaStream_t stream) {
  if (T <= 0 || C <= 0 || R < 0 || (R % 2)) return -6;
  mla_kv_append_kernel<<<T, 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(kv), reinterpret_cast<const __nv_bfloat16*>(gamma),
                                              eps, positions, slots, theta, reinterpret_cast<__nv_bfloat16*>(cache), C, R,
                                              reinterpret_cast<const __nv_bfloat16*>(kidx),
                                              reinterpret_cast<const __nv_bfloat16*>(kidx_gamma),
                                              reinterpret_cast<__nv_bfloat16*>(idx_cache), DI);
  return (int)cudaGetLastError();
}

int b200_mla_q_prepare(const void* q, const int* positions, float theta, void* qn_t, void* q_pe, int T, int H, int N, int R,
                       cudaStream_t stream) {
  if (T <= 0 || H <= 0 || (R % 2)) return -6;
  mla_q_prepare_kernel<<<dim3(T, H), 64, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(q), positions, theta,
                                                      reinterpret_cast<__nv_bfloat16*>(qn_t),
                                                      reinterpret_cast<__nv_bfloat16*>(q_pe), T, H, N, R);
  return (int)cudaGetLastError();
}

int b200_mla_indexer_mma(const void* q_idx, const float* hw, const void* idx_cache, const int* block_table, int max_blocks,
                         int bs, const int* positions, float* scores, int ld, int T, int HI, int DI, float scale,
                         cudaStream_t stream);

// scores fp32 [T, ld]; ld >= max position + 1.  DI must be 32, 64 or 128.
int b200_mla_indexer(const void* q_idx, const float* hw, const void* idx_cache, const int* block_table, int max_blocks, int bs,
                     const int* positions, const int* seq_of_token, float* scores, int ld, int T, int HI, int DI, float scale,
                     cudaStream_t stream) {
  if (T <= 0 || ld <= 0 || HI <= 0) return -6;
  // one sequence, a tensor-core-sized index width and enough queries to fill the 128-query tiles: the tiled kernel
  // (attn_mla_indexer_mma.cu); a decode step (a handful of queries) keeps one thread per key
  if (!seq_of_token && (DI == 64 || DI == 128) && T >= 32)
    return b200_mla_indexer_mma(q_idx, hw, idx_cache, block_table, max_blocks, bs, positions, scores, ld, T, HI, DI, scale, stream);
  const dim3 grid((ld + 127) / 128, T);
  const size_t smem = ((size_t)HI * DI + HI) * sizeof(float);
  auto qp = reinterpret_cast<const __nv_bfloat16*>(q_idx);
  auto kc = reinterpret_cast<const __nv_bfloat16*>(idx_cache);
#define B200_IDX(DI_)                                                                                                  \
  case DI_: {                                                                                                          \
    if (smem > 48 * 1024) cudaFuncSetAttribute(mla_indexer_kernel<DI_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    mla_indexer_kernel<DI_><<<grid, 128, smem, stream>>>(qp, hw, kc, block_table, max_blocks, bs, positions, seq_of_token,  \
                                                         scores, ld, HI, scale);                                      \
    break;                                                                                                             \
  }
  switch (DI) {
    B200_IDX(32)
    B200_IDX(64)
    B200_IDX(128)
    default: return -6;
  }
#undef B200_IDX
  return (int)cudaGetLastError();
}

int b200_topk_rows(const float* vals, int ld, const int* n_valid, int rows, int k, int* idx, cudaStream_t stream) {
  if (rows <= 0 || k <= 0 || ld <= 0) return -6;
  // few rows (decode): one block still owns a row, so give it the largest block
  topk_rows_kernel<<<rows, rows < 296 ? 1024 : 256, 0, stream>>>(vals, ld, n_valid, k, idx);
  return (int)cudaGetLastError();
}

// q_lat [H, T, C], q_pe [T, H, R], cache [rows, C + R]; o_lat [H, T, C].  (C, R) in {(512, 64), (64, 16)}.
int b200_mla_attention_mma(const void* q_lat, const void* q_pe, const void* cache, const int* block_table, int max_blocks,
                           int bs, const int* positions, const int* seq_of_token, const int* sel, int nsel, void* o_lat, int T,
                           int H, int C, int R, float scale, cudaStream_t stream);

// Tensor-core kernel (attn_mla_mma.cu): the heads of a token share one gather of its selected cache rows.
int b200_mla_attention(const void* q_lat, const void* q_pe, const void* cache, const int* block_table, int max_blocks, int bs,
                       const int* positions, const int* seq_of_token, const int* sel, int nsel, void* o_lat, int T, int H, int C,
                       int R, float scale, cudaStream_t stream) {
  return b200_mla_attention_mma(q_lat, q_pe, cache, block_table, max_blocks, bs, positions, seq_of_token, sel, nsel, o_lat, T, H,
                                C, R, scale, stream);
}

// Scalar fp32 kernel, one CTA per (token, head): kept as an independent implementation for cross-checks.
int b200_mla_attention_simt(const void* q_lat, const void* q_pe, const void* cache, const int* block_table, int max_blocks, int bs,
                            const int* positions, const int* seq_of_token, const int* sel, int nsel, void* o_lat, int T, int H,
                            int C, int R, float scale, cudaStream_t stream) {
  if (T <= 0 || H <= 0) return -6;
  auto ql = reinterpret_cast<const __nv_bfloat16*>(q_lat);
  auto qp = reinterpret_cast<const __nv_bfloat16*>(q_pe);
  auto kc = reinterpret_cast<const __nv_bfloat16*>(cache);
  auto ol = reinterpret_cast<__nv_bfloat16*>(o_lat);
  const dim3 grid(T, H);
  if (C == 512 && R == 64)
    mla_attention_kernel<512, 64><<<grid, 128, 0, stream>>>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token,
                                                           sel, nsel, ol, T, H, scale);
  else if (C == 128 && R == 32)
    mla_attention_kernel<128, 32><<<grid, 128, 0, stream>>>(ql, qp, kc, block_table, max_blocks, bs, positions, seq_of_token,
                                                           sel, nsel, ol, T, H, scale);
  else
    return -6;
  return (int)cudaGetLastError();
}

int b200_transpose_heads(const void* in, void* out, int H, int T, int D, cudaStream_t stream) {
  if (H <= 0 || T <= 0 || D <= 0) return -6;
  transpose_heads_kernel<<<dim3(T, H), 128, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(in),
                                                         reinterpret_cast<__nv_bfloat16*>(out), H, T, D);
  return (int)cudaGetLastError();
}

}  // extern "C"
