// Host matrix-vector products straight from raw GGUF blocks (no expansion in memory): y[t, n] = W[n, :] . x[t, :]
// for W stored as Q8_0 (32 values: fp16 scale + 32 int8), IQ2_XXS (codebook magnitudes with sign patterns) or Q2_K (256 values: 16 packed 4-bit scale / 4-bit minimum
// pairs, 64 bytes of 2-bit codes in two 128-value halves of four 32-value planes, fp16 d and dmin; value =
// d * scale * code - dmin * minimum).  Per Q2_K sub-block of 16 the kernel accumulates sum(code * x) and sum(x) and
// applies the two factors once.  Rows are split over host threads; each output is computed by one thread in a fixed
// order.  This is the host path for GGUF routed experts and dense layers of small models.
// Reference behaviour: the Q2_K / Q8_0 row dot kernels of src/csrc/deepseek_cpu_moe_ext.cpp (GGUF raw expert path)
// and the numpy dequantisers they are checked against (src/loader/gguf/tensor_reader.py:258-420).
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <algorithm>
#include <thread>
#include <vector>

namespace {

inline float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1Fu, man = h & 0x3FFu, bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {                                   // subnormal: normalise
      int e = -1;
      do { ++e; man <<= 1; } while (!(man & 0x400u));
      bits = sign | (uint32_t)(127 - 15 - e) << 23 | (man & 0x3FFu) << 13;
    }
  } else if (exp == 31) {
    bits = sign | 0x7F800000u | man << 13;
  } else {
    bits = sign | (exp + 112) << 23 | man << 13;
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

inline uint16_t load_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }

float dot_q8_0(const uint8_t* row, const float* x, int k) {
  float total = 0.f;
  for (int b = 0; b < k / 32; ++b) {
    const uint8_t* blk = row + (size_t)b * 34;
    const int8_t* q = reinterpret_cast<const int8_t*>(blk + 2);
    const float* xb = x + b * 32;
    float acc = 0.f;
    for (int i = 0; i < 32; ++i) acc += (float)q[i] * xb[i];
    total += acc * half_to_float(load_u16(blk));
  }
  return total;
}

float dot_q2_k(const uint8_t* row, const float* x, int k) {
  float total = 0.f;
  for (int b = 0; b < k / 256; ++b) {
    const uint8_t* blk = row + (size_t)b * 84;
    const uint8_t* scales = blk;
    const uint8_t* qs = blk + 16;
    const float d = half_to_float(load_u16(blk + 80)), dmin = half_to_float(load_u16(blk + 82));
    const float* xb = x + b * 256;
    float acc = 0.f;
    for (int half = 0; half < 2; ++half)
      for (int plane = 0; plane < 4; ++plane)
        for (int part = 0; part < 2; ++part) {                 // 16 values share a scale / minimum
          const int base = half * 128 + plane * 32 + part * 16;
          const uint8_t* q = qs + half * 32 + part * 16;
          float sq = 0.f, sx = 0.f;
          for (int i = 0; i < 16; ++i) {
            const float xv = xb[base + i];
            sq += (float)((q[i] >> (2 * plane)) & 3) * xv;
            sx += xv;
          }
          const uint8_t sc = scales[base / 16];
          acc += d * (float)(sc & 0x0F) * sq - dmin * (float)(sc >> 4) * sx;
        }
    total += acc;
  }
  return total;
}

// IQ2_XXS: 256 values = fp16 d + eight 8-byte groups of 32 values: four codebook indices (8 magnitudes each), then a word
// holding four 7-bit sign-pattern indices and a 4-bit scale; value = d * (0.5 + scale) / 4 * magnitude * sign.
// The codebook is not compiled in: the loader hands it over once.
float g_iq2xxs_grid[256 * 8];
float g_sign_rows[128 * 8];          // +1 / -1 per value for every sign pattern, so the inner loop is a plain 8-wide FMA
bool g_iq2xxs_ready = false;

float dot_iq2_xxs(const uint8_t* row, const float* x, int k) {
  float total = 0.f;
  for (int b = 0; b < k / 256; ++b) {
    const uint8_t* blk = row + (size_t)b * 66;
    const float d = half_to_float(load_u16(blk));
    const float* xb = x + b * 256;
    for (int g = 0; g < 8; ++g) {
      const uint8_t* q = blk + 2 + g * 8;
      uint32_t w1;
      memcpy(&w1, q + 4, 4);
      const float db = d * (0.5f + (float)(w1 >> 28)) * 0.25f;
      float acc = 0.f;
      for (int j = 0; j < 4; ++j) {
        const float* mag = g_iq2xxs_grid + (size_t)q[j] * 8;
        const float* sg = g_sign_rows + (size_t)((w1 >> (7 * j)) & 0x7F) * 8;
        const float* xv = xb + g * 32 + j * 8;
        for (int i = 0; i < 8; ++i) acc += mag[i] * sg[i] * xv[i];
      }
      total += db * acc;
    }
  }
  return total;
}

template <class F>
void parallel_rows(long long n, int requested, F fn) {
  int nt = requested > 0 ? requested : (int)std::thread::hardware_concurrency();
  nt = std::max(1, std::min(nt, 64));
  if ((long long)nt > n / 16) nt = (int)std::max<long long>(1, n / 16);
  if (nt <= 1) {
    fn(0, n);
    return;
  }
  std::vector<std::thread> pool;
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

// The IQ2_XXS codebook (256 x 8 magnitudes) and the 128 sign patterns; call once before using type 16.
void b200_cpu_gguf_set_iq2xxs_tables(const float* grid, const uint8_t* ksigns) {
  memcpy(g_iq2xxs_grid, grid, sizeof(g_iq2xxs_grid));
  for (int p = 0; p < 128; ++p)
    for (int i = 0; i < 8; ++i) g_sign_rows[p * 8 + i] = (ksigns[p] >> i) & 1 ? -1.f : 1.f;
  g_iq2xxs_ready = true;
}

// ggml_type 8 = Q8_0 (K % 32 == 0), 10 = Q2_K (K % 256 == 0), 16 = IQ2_XXS (K % 256 == 0, tables set: else -3).  x [T, K] fp32, raw [N, row_bytes] as in the file,
// y [T, N] fp32 (overwritten).  Returns 0, -1 on a bad shape, -2 on an unsupported type.
int b200_cpu_gguf_linear(int ggml_type, const float* x, int T, int K, const uint8_t* raw, int N, float* y, int num_threads) {
  if (T <= 0 || K <= 0 || N <= 0) return -1;
  size_t row_bytes;
  if (ggml_type == 8) {
    if (K % 32) return -1;
    row_bytes = (size_t)K / 32 * 34;
  } else if (ggml_type == 10) {
    if (K % 256) return -1;
    row_bytes = (size_t)K / 256 * 84;
  } else if (ggml_type == 16) {
    if (K % 256) return -1;
    if (!g_iq2xxs_ready) return -3;
    row_bytes = (size_t)K / 256 * 66;
  } else {
    return -2;
  }
  parallel_rows((long long)T * N, num_threads, [&](long long lo, long long hi) {
    for (long long u = lo; u < hi; ++u) {
      const size_t t = (size_t)(u / N), n = (size_t)(u % N);
      const uint8_t* row = raw + n * row_bytes;
      const float* xr = x + t * (size_t)K;
      y[u] = ggml_type == 8 ? dot_q8_0(row, xr, K) : ggml_type == 10 ? dot_q2_k(row, xr, K) : dot_iq2_xxs(row, xr, K);
    }
  });
  return 0;
}

}  // extern "C"
