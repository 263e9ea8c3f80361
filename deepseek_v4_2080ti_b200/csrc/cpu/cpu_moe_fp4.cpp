// CPU routed-expert MoE on raw FP4 weights (E2M1 nibbles, low nibble first, one UE8M0 scale per 32
// inputs): y[t] += sum_k w[t,k] * W2_e( silu(W1_e x[t]) * (W3_e x[t]) ),  e = idx[t,k].
// The packed bytes are decoded 32 elements at a time in registers (pshufb lookup of 2*level, then
// int8 -> fp32 and FMA); the weights are never expanded in memory.  Work is split over host threads
// in two phases (expert hidden rows, then output rows) with a fixed summation order, so results do
// not depend on the thread count.
// This is the CPU oracle / small-model path; it mirrors what the reference's AVX2 extension does for
// raw FP4 experts (src/csrc/deepseek_cpu_moe_ext.cpp:1778-1886).
#include <immintrin.h>
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

namespace {

// 2 * level for every 4-bit code; the factor 0.5 is folded into the group scale.
alignas(16) const int8_t kLut2x[16] = {0, 1, 2, 3, 4, 6, 8, 12, 0, -1, -2, -3, -4, -6, -8, -12};

inline float e8m0_half(uint8_t e) {
  // 0.5 * 2^(e - 127)
  return ldexpf(0.5f, (int)e - 127);
}

inline float hsum256(__m256 v) {
  __m128 lo = _mm256_castps256_ps128(v), hi = _mm256_extractf128_ps(v, 1);
  lo = _mm_add_ps(lo, hi);
  lo = _mm_hadd_ps(lo, lo);
  lo = _mm_hadd_ps(lo, lo);
  return _mm_cvtss_f32(lo);
}

// dot(row, x) for one packed row of `n` elements (n % 32 == 0).
float dot_fp4_row(const uint8_t* w, const uint8_t* s, const float* x, int n) {
  const __m128i lut = _mm_load_si128(reinterpret_cast<const __m128i*>(kLut2x));
  const __m128i mask = _mm_set1_epi8(0x0F);
  float total = 0.f;
  for (int g = 0; g < n / 32; ++g) {
    const __m128i bytes = _mm_loadu_si128(reinterpret_cast<const __m128i*>(w + g * 16));
    const __m128i lo = _mm_shuffle_epi8(lut, _mm_and_si128(bytes, mask));                      // elements 0,2,4,...
    const __m128i hi = _mm_shuffle_epi8(lut, _mm_and_si128(_mm_srli_epi16(bytes, 4), mask));   // elements 1,3,5,...
    const __m128i e0 = _mm_unpacklo_epi8(lo, hi);   // elements 0..15
    const __m128i e1 = _mm_unpackhi_epi8(lo, hi);   // elements 16..31
    const float* xg = x + g * 32;
    __m256 acc = _mm256_mul_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(e0)), _mm256_loadu_ps(xg));
    acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_srli_si128(e0, 8))), _mm256_loadu_ps(xg + 8), acc);
    acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(e1)), _mm256_loadu_ps(xg + 16), acc);
    acc = _mm256_fmadd_ps(_mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(_mm_srli_si128(e1, 8))), _mm256_loadu_ps(xg + 24), acc);
    total += hsum256(acc) * e8m0_half(s[g]);
  }
  return total;
}

inline float silu(float v) { return v / (1.f + expf(-v)); }

int resolve_threads(int requested, long long work) {
  int nt = requested > 0 ? requested : (int)std::thread::hardware_concurrency();
  if (nt < 1) nt = 1;
  if (nt > 64) nt = 64;
  if ((long long)nt > work) nt = (int)std::max<long long>(1, work);
  return nt;
}

// Static contiguous partition of [0, n) over nt threads; fn(begin, end).
template <class F>
void parallel_for(long long n, int nt, F fn) {
  if (nt <= 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> pool;
  pool.reserve(nt - 1);
  const long long per = (n + nt - 1) / nt;
  for (int i = 1; i < nt; ++i) {
    const long long b = std::min(n, i * per), e = std::min(n, (i + 1) * per);
    if (b < e) pool.emplace_back([=] { fn(b, e); });
  }
  fn(0, std::min(n, per));
  for (auto& t : pool) t.join();
}

}  // namespace

extern "C" {

// x [T, H] fp32; topk_idx [T, K] int32 (negative = unused route); topk_w [T, K] fp32;
// w13 [E, 2I, H/2] + s13 [E, 2I, H/32] (rows 0..I-1 gate, I..2I-1 up); w2 [E, H, I/2] + s2 [E, H, I/32];
// out [T, H] fp32 is incremented.  H % 32 == 0, I % 32 == 0.  Returns 0, or -1 on a bad argument.
int b200_cpu_moe_fp4_forward(const float* x, int T, int H, const int* topk_idx, const float* topk_w, int K,
                             const uint8_t* w13, const uint8_t* s13, const uint8_t* w2, const uint8_t* s2, int E,
                             int I, float swiglu_limit, float* out, int num_threads) {
  if (T <= 0 || H <= 0 || I <= 0 || K <= 0 || (H % 32) || (I % 32)) return -1;
  for (int r = 0; r < T * K; ++r)
    if (topk_idx[r] >= E) return -1;
  const size_t R = (size_t)T * K;
  std::vector<float> hidden(R * I);
  const size_t w13_e = (size_t)2 * I * (H / 2), s13_e = (size_t)2 * I * (H / 32);
  const size_t w2_e = (size_t)H * (I / 2), s2_e = (size_t)H * (I / 32);
  // phase 1: hidden[r, i] = w[r] * silu(gate) * up
  const long long n1 = (long long)R * I;
  parallel_for(n1, resolve_threads(num_threads, n1 / 64), [&](long long lo, long long hi) {
  for (long long u = lo; u < hi; ++u) {
    const size_t r = (size_t)(u / I);
    const int i = (int)(u % I);
    const int e = topk_idx[r];
    if (e < 0) {
      hidden[u] = 0.f;
      continue;
    }
    const float* xr = x + (r / K) * (size_t)H;
    float gate = dot_fp4_row(w13 + e * w13_e + (size_t)i * (H / 2), s13 + e * s13_e + (size_t)i * (H / 32), xr, H);
    float up = dot_fp4_row(w13 + e * w13_e + (size_t)(I + i) * (H / 2), s13 + e * s13_e + (size_t)(I + i) * (H / 32), xr, H);
    if (swiglu_limit > 0.f) {
      up = fminf(fmaxf(up, -swiglu_limit), swiglu_limit);
      gate = fminf(gate, swiglu_limit);
    }
    hidden[u] = topk_w[r] * silu(gate) * up;
  }
  });
  // phase 2: out[t, h] += sum_k W2_e[h, :] . hidden[t*K + k, :]   (k ascending)
  const long long n2 = (long long)T * H;
  parallel_for(n2, resolve_threads(num_threads, n2 / 64), [&](long long lo, long long hi) {
  for (long long u = lo; u < hi; ++u) {
    const size_t t = (size_t)(u / H);
    const int h = (int)(u % H);
    float acc = 0.f;
    for (int k = 0; k < K; ++k) {
      const int e = topk_idx[t * K + k];
      if (e < 0) continue;
      acc += dot_fp4_row(w2 + e * w2_e + (size_t)h * (I / 2), s2 + e * s2_e + (size_t)h * (I / 32),
                         hidden.data() + (t * K + k) * (size_t)I, I);
    }
    out[u] += acc;
  }
  });
  return 0;
}

// y [T, N] = x [T, Kdim] * W^T for one FP4 matrix W [N, Kdim/2] + scales [N, Kdim/32] (dense layers, tests).
int b200_cpu_fp4_linear(const float* x, int T, int Kdim, const uint8_t* w, const uint8_t* s, int N, float* y,
                        int num_threads) {
  if (T <= 0 || N <= 0 || Kdim <= 0 || (Kdim % 32)) return -1;
  const long long n = (long long)T * N;
  parallel_for(n, resolve_threads(num_threads, n / 64), [&](long long lo, long long hi) {
  for (long long u = lo; u < hi; ++u) {
    const size_t t = (size_t)(u / N);
    const int r = (int)(u % N);
    y[u] = dot_fp4_row(w + (size_t)r * (Kdim / 2), s + (size_t)r * (Kdim / 32), x + t * (size_t)Kdim, Kdim);
  }
  });
  return 0;
}

}  // extern "C"
