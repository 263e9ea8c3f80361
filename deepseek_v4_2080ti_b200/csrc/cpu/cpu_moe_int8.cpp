// CPU routed-expert MoE on INT8 weights with one fp32 scale per output row (W8A8): activations are quantised per
// token to int8 (scale = max|x| / 127, round to nearest even), every row product is an exact int32 dot product
// (sign-extend to int16, multiply, pairwise add) scaled once by a_scale * w_scale[row].  The SwiGLU output of each
// route is quantised again the same way before the down projection.
//   y[t] += sum_k w[t,k] * W2_e( silu(W1_e x[t]) * (W3_e x[t]) ),  e = idx[t,k]
// Work is split over host threads in two phases with a fixed summation order, so results do not depend on the
// thread count, and because the dot products are integer the result equals a straightforward reference bit for bit
// up to the final fp32 scaling.
// Reference behaviour: the INT8 per-row routed forward of src/csrc/deepseek_cpu_moe_ext.cpp:2000-2200 and its int8
// dot kernels :540-660.
#include <immintrin.h>
#include <math.h>
#include <stdint.h>

#include <algorithm>
#include <thread>
#include <vector>

namespace {

inline int32_t hsum_epi32(__m256i v) {
  __m128i lo = _mm256_castsi256_si128(v), hi = _mm256_extracti128_si256(v, 1);
  lo = _mm_add_epi32(lo, hi);
  lo = _mm_hadd_epi32(lo, lo);
  lo = _mm_hadd_epi32(lo, lo);
  return _mm_cvtsi128_si32(lo);
}

// exact sum_i a[i] * b[i] over int8 vectors, n % 16 == 0 handled by the vector loop, the rest scalar
int32_t dot_i8(const int8_t* a, const int8_t* b, int n) {
  __m256i acc = _mm256_setzero_si256();
  int i = 0;
  for (; i + 16 <= n; i += 16) {
    const __m256i va = _mm256_cvtepi8_epi16(_mm_loadu_si128(reinterpret_cast<const __m128i*>(a + i)));
    const __m256i vb = _mm256_cvtepi8_epi16(_mm_loadu_si128(reinterpret_cast<const __m128i*>(b + i)));
    acc = _mm256_add_epi32(acc, _mm256_madd_epi16(va, vb));
  }
  int32_t total = hsum_epi32(acc);
  for (; i < n; ++i) total += (int32_t)a[i] * (int32_t)b[i];
  return total;
}

// q = round_to_nearest_even(x / scale) clamped to [-127, 127]; returns scale (0 for an all-zero row)
float quantize_row(const float* x, int n, int8_t* q) {
  float amax = 0.f;
  for (int i = 0; i < n; ++i) amax = fmaxf(amax, fabsf(x[i]));
  if (amax == 0.f) {
    std::fill(q, q + n, (int8_t)0);
    return 0.f;
  }
  const float scale = amax / 127.f;
  for (int i = 0; i < n; ++i) {
    const float v = nearbyintf(x[i] / scale);
    q[i] = (int8_t)fminf(fmaxf(v, -127.f), 127.f);
  }
  return scale;
}

inline float silu(float v) { return v / (1.f + expf(-v)); }

int resolve_threads(int requested, long long work) {
  int nt = requested > 0 ? requested : (int)std::thread::hardware_concurrency();
  nt = std::max(1, std::min(nt, 64));
  if ((long long)nt > work) nt = (int)std::max<long long>(1, work);
  return nt;
}

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
// w13 int8 [E, 2I, H] + s13 fp32 [E, 2I] (rows 0..I-1 gate, I..2I-1 up); w2 int8 [E, H, I] + s2 fp32 [E, H];
// out [T, H] fp32 is incremented.  Returns 0, or -1 on a bad argument.
int b200_cpu_moe_int8_forward(const float* x, int T, int H, const int* topk_idx, const float* topk_w, int K,
                              const int8_t* w13, const float* s13, const int8_t* w2, const float* s2, int E, int I,
                              float swiglu_limit, float* out, int num_threads) {
  if (T <= 0 || H <= 0 || I <= 0 || K <= 0 || E <= 0) return -1;
  for (int r = 0; r < T * K; ++r)
    if (topk_idx[r] >= E) return -1;
  const size_t R = (size_t)T * K;
  std::vector<int8_t> xq((size_t)T * H);
  std::vector<float> xs(T);
  parallel_for(T, resolve_threads(num_threads, T), [&](long long lo, long long hi) {
    for (long long t = lo; t < hi; ++t) xs[t] = quantize_row(x + t * (size_t)H, H, xq.data() + t * (size_t)H);
  });
  std::vector<float> hidden(R * I);
  const size_t w13_e = (size_t)2 * I * H, w2_e = (size_t)H * I;
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
      const size_t t = r / K;
      const int8_t* xr = xq.data() + t * (size_t)H;
      float gate = (float)dot_i8(w13 + e * w13_e + (size_t)i * H, xr, H) * (xs[t] * s13[(size_t)e * 2 * I + i]);
      float up = (float)dot_i8(w13 + e * w13_e + (size_t)(I + i) * H, xr, H) * (xs[t] * s13[(size_t)e * 2 * I + I + i]);
      if (swiglu_limit > 0.f) {
        up = fminf(fmaxf(up, -swiglu_limit), swiglu_limit);
        gate = fminf(gate, swiglu_limit);
      }
      hidden[u] = topk_w[r] * silu(gate) * up;
    }
  });
  // re-quantise every route's hidden row for the down projection
  std::vector<int8_t> hq(R * I);
  std::vector<float> hs(R);
  parallel_for((long long)R, resolve_threads(num_threads, (long long)R), [&](long long lo, long long hi) {
    for (long long r = lo; r < hi; ++r) hs[r] = quantize_row(hidden.data() + r * (size_t)I, I, hq.data() + r * (size_t)I);
  });
  // phase 2: out[t, h] += sum_k W2_e[h, :] . hidden[t*K + k, :]   (k ascending)
  const long long n2 = (long long)T * H;
  parallel_for(n2, resolve_threads(num_threads, n2 / 64), [&](long long lo, long long hi) {
    for (long long u = lo; u < hi; ++u) {
      const size_t t = (size_t)(u / H);
      const int h = (int)(u % H);
      float acc = 0.f;
      for (int k = 0; k < K; ++k) {
        const size_t r = t * K + k;
        const int e = topk_idx[r];
        if (e < 0) continue;
        acc += (float)dot_i8(w2 + e * w2_e + (size_t)h * I, hq.data() + r * (size_t)I, I) * (hs[r] * s2[(size_t)e * H + h]);
      }
      out[u] += acc;
    }
  });
  return 0;
}

// Per-row symmetric INT8 quantisation of a weight matrix w [N, K] fp32 -> q int8 [N, K], scale fp32 [N].
int b200_cpu_quantize_rows_int8(const float* w, int N, int K, int8_t* q, float* scale, int num_threads) {
  if (N <= 0 || K <= 0) return -1;
  parallel_for(N, resolve_threads(num_threads, N), [&](long long lo, long long hi) {
    for (long long r = lo; r < hi; ++r) scale[r] = quantize_row(w + r * (size_t)K, K, q + r * (size_t)K);
  });
  return 0;
}

}  // extern "C"
