// Memory-safety self-test of the AVX2 host kernels (csrc/cpu), meant for -fsanitize=address,undefined: every operand
// sits in a heap block of exactly its size, so a vector load or store that runs past a row's end lands in a redzone.
// Shapes are the smallest legal ones and a few odd multiples; refused arguments must be refused before any access.
// Results are compared with plain scalar arithmetic where that is cheap.  Exit code 0 = every check held.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

extern "C" {
int b200_cpu_moe_fp4_forward(const float* x, int T, int H, const int* topk_idx, const float* topk_w, int K, const uint8_t* w13,
                             const uint8_t* s13, const uint8_t* w2, const uint8_t* s2, int E, int I, float swiglu_limit,
                             float* out, int num_threads);
int b200_cpu_fp4_linear(const float* x, int T, int Kdim, const uint8_t* w, const uint8_t* s, int N, float* y, int num_threads);
int b200_cpu_moe_int8_forward(const float* x, int T, int H, const int* topk_idx, const float* topk_w, int K, const int8_t* w13,
                              const float* s13, const int8_t* w2, const float* s2, int E, int I, float swiglu_limit, float* out,
                              int num_threads);
int b200_cpu_quantize_rows_int8(const float* w, int N, int K, int8_t* q, float* scale, int num_threads);
int b200_cpu_gguf_linear(int ggml_type, const float* x, int T, int K, const uint8_t* raw, int N, float* y, int num_threads);
}

static int g_fail = 0;
#define CHECK(cond)                                                                                          \
  do {                                                                                                       \
    if (!(cond)) { std::fprintf(stderr, "CHECK failed %s:%d: %s\n", __FILE__, __LINE__, #cond); ++g_fail; }  \
  } while (0)

static std::mt19937 rng(17);

// heap block of exactly n elements (never a vector with spare capacity)
template <class T> struct Exact {
  T* p;
  size_t n;
  explicit Exact(size_t n_) : p(static_cast<T*>(std::malloc(n_ ? n_ * sizeof(T) : 1))), n(n_) {}
  ~Exact() { std::free(p); }
  Exact(const Exact&) = delete;
  T& operator[](size_t i) { return p[i]; }
};

static void fill_f(Exact<float>& a, float scale = 1.f) {
  std::normal_distribution<float> d(0.f, scale);
  for (size_t i = 0; i < a.n; ++i) a[i] = d(rng);
}
template <class T> static void fill_bytes(Exact<T>& a, int lo, int hi) {
  for (size_t i = 0; i < a.n; ++i) a[i] = T(lo + int(rng() % unsigned(hi - lo + 1)));
}

static void test_fp4() {
  for (int H : {32, 96}) for (int I : {32, 64}) for (int T : {1, 3}) {
    const int E = 3, K = 2;
    Exact<float> x(size_t(T) * H), w(size_t(T) * K), out(size_t(T) * H);
    Exact<int> idx(size_t(T) * K);
    Exact<uint8_t> w13(size_t(E) * 2 * I * (H / 2)), s13(size_t(E) * 2 * I * (H / 32)), w2(size_t(E) * H * (I / 2)), s2(size_t(E) * H * (I / 32));
    fill_f(x); fill_f(w, 0.5f);
    fill_bytes(w13, 0, 255); fill_bytes(w2, 0, 255);
    fill_bytes(s13, 120, 130); fill_bytes(s2, 120, 130);            // UE8M0 exponents near 1.0
    for (size_t i = 0; i < idx.n; ++i) idx[i] = int(rng() % (E + 1)) - 1;       // -1 = unused route
    std::memset(out.p, 0, out.n * sizeof(float));
    CHECK(b200_cpu_moe_fp4_forward(x.p, T, H, idx.p, w.p, K, w13.p, s13.p, w2.p, s2.p, E, I, 7.f, out.p, 2) == 0);
    for (size_t i = 0; i < out.n; ++i) CHECK(std::isfinite(out[i]));
    idx[0] = E;                                                      // a route to an expert that does not exist
    CHECK(b200_cpu_moe_fp4_forward(x.p, T, H, idx.p, w.p, K, w13.p, s13.p, w2.p, s2.p, E, I, 7.f, out.p, 2) == -1);
  }
  CHECK(b200_cpu_moe_fp4_forward(nullptr, 1, 48, nullptr, nullptr, 1, nullptr, nullptr, nullptr, nullptr, 1, 32, 0.f, nullptr, 1) == -1);
  for (int Kd : {32, 160}) for (int N : {1, 5}) {
    Exact<float> x(size_t(2) * Kd), y(size_t(2) * N);
    Exact<uint8_t> w(size_t(N) * (Kd / 2)), s(size_t(N) * (Kd / 32));
    fill_f(x); fill_bytes(w, 0, 255); fill_bytes(s, 125, 129);
    CHECK(b200_cpu_fp4_linear(x.p, 2, Kd, w.p, s.p, N, y.p, 3) == 0);
    for (size_t i = 0; i < y.n; ++i) CHECK(std::isfinite(y[i]));
  }
  CHECK(b200_cpu_fp4_linear(nullptr, 1, 40, nullptr, nullptr, 1, nullptr, 1) == -1);
}

static void test_int8() {
  for (int H : {8, 40, 64}) for (int I : {8, 24}) for (int T : {1, 2}) {
    const int E = 2, K = 2;
    Exact<float> x(size_t(T) * H), w(size_t(T) * K), out(size_t(T) * H), s13(size_t(E) * 2 * I), s2(size_t(E) * H);
    Exact<int> idx(size_t(T) * K);
    Exact<int8_t> w13(size_t(E) * 2 * I * H), w2(size_t(E) * H * I);
    fill_f(x); fill_f(w, 0.5f);
    fill_bytes(w13, -127, 127); fill_bytes(w2, -127, 127);
    for (size_t i = 0; i < s13.n; ++i) s13[i] = 0.01f;
    for (size_t i = 0; i < s2.n; ++i) s2[i] = 0.01f;
    for (size_t i = 0; i < idx.n; ++i) idx[i] = int(rng() % (E + 1)) - 1;
    std::memset(out.p, 0, out.n * sizeof(float));
    CHECK(b200_cpu_moe_int8_forward(x.p, T, H, idx.p, w.p, K, w13.p, s13.p, w2.p, s2.p, E, I, 0.f, out.p, 2) == 0);
    for (size_t i = 0; i < out.n; ++i) CHECK(std::isfinite(out[i]));
  }
  for (int N : {1, 3}) for (int Kd : {1, 7, 33}) {
    Exact<float> wf(size_t(N) * Kd), sc(N);
    Exact<int8_t> q(size_t(N) * Kd);
    fill_f(wf);
    CHECK(b200_cpu_quantize_rows_int8(wf.p, N, Kd, q.p, sc.p, 2) == 0);
    for (int r = 0; r < N; ++r)
      for (int c = 0; c < Kd; ++c) CHECK(std::fabs(q[size_t(r) * Kd + c] * sc[r] - wf[size_t(r) * Kd + c]) <= sc[r] * 0.51f + 1e-6f);
  }
}

static void test_gguf() {
  // Q8_0: 34-byte blocks (fp16 scale + 32 int8); compare with scalar arithmetic
  for (int Kd : {32, 96}) for (int N : {1, 4}) {
    const int T = 2;
    Exact<float> x(size_t(T) * Kd), y(size_t(T) * N);
    Exact<uint8_t> raw(size_t(N) * (Kd / 32) * 34);
    fill_f(x);
    for (size_t b = 0; b < raw.n / 34; ++b) {
      raw[b * 34] = 0x00; raw[b * 34 + 1] = 0x2C;                  // fp16 0x2C00 = 0.0625
      for (int i = 0; i < 32; ++i) raw[b * 34 + 2 + i] = uint8_t(int8_t(int(rng() % 255) - 127));
    }
    CHECK(b200_cpu_gguf_linear(8, x.p, T, Kd, raw.p, N, y.p, 2) == 0);
    for (int t = 0; t < T; ++t)
      for (int n = 0; n < N; ++n) {
        double want = 0;
        for (int k = 0; k < Kd; ++k) want += 0.0625 * int8_t(raw[(size_t(n) * (Kd / 32) + k / 32) * 34 + 2 + k % 32]) * x[size_t(t) * Kd + k];
        CHECK(std::fabs(y[size_t(t) * N + n] - want) < 1e-3 * (1.0 + std::fabs(want)));
      }
  }
  // Q2_K: 84-byte blocks of 256 values; arbitrary bytes with a small fp16 scale pair at the end
  for (int N : {1, 3}) {
    const int Kd = 256, T = 1;
    Exact<float> x(size_t(T) * Kd), y(size_t(T) * N);
    Exact<uint8_t> raw(size_t(N) * 84);
    fill_f(x); fill_bytes(raw, 0, 255);
    for (int n = 0; n < N; ++n) { raw[size_t(n) * 84 + 80] = 0x00; raw[size_t(n) * 84 + 81] = 0x2C; raw[size_t(n) * 84 + 82] = 0x00; raw[size_t(n) * 84 + 83] = 0x2C; }
    CHECK(b200_cpu_gguf_linear(10, x.p, T, Kd, raw.p, N, y.p, 2) == 0);
    for (size_t i = 0; i < y.n; ++i) CHECK(std::isfinite(y[i]));
  }
  CHECK(b200_cpu_gguf_linear(8, nullptr, 1, 33, nullptr, 1, nullptr, 1) == -1);
  CHECK(b200_cpu_gguf_linear(10, nullptr, 1, 128, nullptr, 1, nullptr, 1) == -1);
  CHECK(b200_cpu_gguf_linear(16, nullptr, 1, 256, nullptr, 1, nullptr, 1) == -3);          // codebook tables not set
  CHECK(b200_cpu_gguf_linear(99, nullptr, 1, 256, nullptr, 1, nullptr, 1) == -2);
}

int main() {
  test_fp4();
  test_int8();
  test_gguf();
  if (g_fail) { std::fprintf(stderr, "%d check(s) failed\n", g_fail); return 1; }
  std::puts("CPU_SELFTEST_OK");
  return 0;
}
