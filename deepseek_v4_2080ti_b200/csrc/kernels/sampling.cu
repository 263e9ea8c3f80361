// Token sampling on the device: temperature, top-k, top-p (nucleus) and min-p over a candidate set, plus repetition /
// presence / frequency penalties applied to the logits beforehand.
//
// The candidate set of a row is its K largest logits (K = top_k, or 1024 when top-k is off: the tail beyond the 1024
// most likely tokens carries no mass that nucleus sampling would keep), found by the radix select of attn_mla.cu
// (b200_topk_rows).  One CTA per row then sorts the candidates, forms the tempered softmax over them, cuts by top-p
// and min-p, renormalises and draws with a caller-supplied uniform number, so a run is reproducible from its seed.
// With a vocabulary sharded over ranks, every rank selects candidates from its shard, the (value, id) pairs are
// gathered and this kernel runs on the merged list.
//
// Reference behaviour: logit processors + Gumbel-max sampling (src/models/deepseek_v4/generation.py:40-220) and the
// native sampler ops (cpp_engine/include/sampler_ops.hpp, backends/cuda/kernels/sampler_ops.cu).
#include <cuda_runtime.h>
#include <stdint.h>
#include "ops.h"

namespace {

constexpr int KMAX = 1024;

// vals: [rows, ld] fp32; idx: [rows, K] positions into the row (-1 = empty).  out_pos: chosen position per row.
__global__ void __launch_bounds__(256)
sample_candidates_kernel(const float* __restrict__ vals, int ld, const int* __restrict__ idx, int K, float temperature,
                         float top_p, float min_p, const float* __restrict__ u, int* __restrict__ out_pos,
                         float* __restrict__ out_prob) {
  __shared__ float sv[KMAX];
  __shared__ int si[KMAX];
  __shared__ float red[8];
  const int row = blockIdx.x, tid = threadIdx.x;
  const float* v = vals + (size_t)row * ld;
  const int* ix = idx + (size_t)row * K;
  int kp = 1;
  while (kp < K) kp <<= 1;
  for (int i = tid; i < kp; i += 256) {
    const int p = i < K ? ix[i] : -1;
    si[i] = p;
    sv[i] = p >= 0 ? v[p] : -INFINITY;
  }
  __syncthreads();
  // bitonic sort, descending by value, ties by ascending position (deterministic)
  for (int size = 2; size <= kp; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < kp / 2; i += 256) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool desc = ((lo & size) == 0);
        const float a = sv[lo], b = sv[hi];
        const int ia = si[lo], ib = si[hi];
        const bool a_first = (a > b) || (a == b && (unsigned)ia < (unsigned)ib);   // -1 sorts last
        if (a_first != desc) {
          sv[lo] = b; sv[hi] = a;
          si[lo] = ib; si[hi] = ia;
        }
      }
      __syncthreads();
    }
  }
  const float vmax = sv[0];
  __syncthreads();   // every thread holds the top logit before the loop below overwrites sv[] in place
  const float inv_t = 1.f / temperature;
  // tempered softmax numerators
  float part = 0.f;
  for (int i = tid; i < kp; i += 256) {
    const float e = si[i] >= 0 ? __expf((sv[i] - vmax) * inv_t) : 0.f;
    sv[i] = e;
    part += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
  if ((tid & 31) == 0) red[tid >> 5] = part;
  __syncthreads();
  float total = 0.f;
  for (int w = 0; w < 8; ++w) total += red[w];
  // the cuts and the draw walk the sorted list once: K <= 1024, one thread
  if (tid == 0) {
    const float pmax = sv[0] / total;
    float cum = 0.f;
    int n = 0;
    for (; n < kp && si[n] >= 0; ++n) {
      const float pr = sv[n] / total;
      if (n > 0 && (pr < min_p * pmax || cum >= top_p)) break;
      cum += pr;
    }
    // draw inside the kept mass
    const float target = u[row] * cum;
    float acc = 0.f;
    int pick = 0;
    for (int i = 0; i < n; ++i) {
      acc += sv[i] / total;
      pick = i;
      if (acc > target) break;
    }
    out_pos[row] = si[pick];
    if (out_prob) out_prob[row] = (sv[pick] / total) / cum;
  }
}

// logits[row, id] adjusted in place for every id of the row's history: repetition (divide positive / multiply negative
// logits), presence (flat) and frequency (per occurrence) penalties.  counts: int32 [rows, n] occurrences, or null.
__global__ void penalties_kernel(float* __restrict__ logits, int ld, int n, const int* __restrict__ counts, float repetition,
                                 float presence, float frequency) {
  const int row = blockIdx.y;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int c = counts[(size_t)row * n + i];
  if (c <= 0) return;
  float x = logits[(size_t)row * ld + i];
  if (repetition != 1.f) x = x > 0.f ? x / repetition : x * repetition;
  x -= presence + frequency * (float)c;
  logits[(size_t)row * ld + i] = x;
}

}  // namespace

extern "C" {

// Draw one candidate per row.  vals fp32 [rows, ld]; idx int32 [rows, K] positions into the row, -1 = empty, K <= 1024;
// u fp32 [rows] uniforms in [0, 1); out_pos int32 [rows]; out_prob (optional) the renormalised probability of the draw.
int b200_sample_candidates(const float* vals, int ld, const int* idx, int K, int rows, float temperature, float top_p,
                           float min_p, const float* u, int* out_pos, float* out_prob, cudaStream_t stream) {
  if (rows <= 0 || K <= 0 || K > KMAX || temperature <= 0.f || top_p <= 0.f) return -6;
  sample_candidates_kernel<<<rows, 256, 0, stream>>>(vals, ld, idx, K, temperature, top_p, min_p, u, out_pos, out_prob);
  return (int)cudaGetLastError();
}

int b200_apply_penalties(float* logits, int ld, int n, int rows, const int* counts, float repetition, float presence,
                         float frequency, cudaStream_t stream) {
  if (rows <= 0 || n <= 0 || !counts || repetition <= 0.f) return -6;
  penalties_kernel<<<dim3((n + 255) / 256, rows), 256, 0, stream>>>(logits, ld, n, counts, repetition, presence, frequency);
  return (int)cudaGetLastError();
}

}  // extern "C"
