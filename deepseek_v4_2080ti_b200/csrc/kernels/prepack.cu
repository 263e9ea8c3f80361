// Device-side weight preparation used by the native engine at load time:
//   prepack_fp8   - FP8 [N, K] row-major -> the GEMM's tile-major layout [ceil(N/128)][ceil(K/64)][128 rows][64 bytes]
//                   with each 4-byte group stored as (w0, w2, w1, w3) and the 16-byte chunks of row r at chunk index
//                   c ^ ((r >> 1) & 3) (same transformation as ops/gemm.py:prepack_fp8);
//   bf16_to_f32   - block scales and per-head constants come as bf16 in the checkpoint, the kernels read fp32.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include "ops.h"

namespace {

__global__ void prepack_fp8_kernel(const uint8_t* __restrict__ w, uint8_t* __restrict__ out, int N, int K, int kb_total) {
  // one thread per output 4-byte group
  const size_t gid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t groups_per_tile = 128 * 16;
  const size_t total = (size_t)((N + 127) / 128) * kb_total * groups_per_tile;
  if (gid >= total) return;
  const size_t tile = gid / groups_per_tile;
  const int in_tile = (int)(gid % groups_per_tile);
  const int r = in_tile / 16, g = in_tile % 16;          // row in tile, physical 4-byte group in the 64-byte row
  const int pc = g / 4, gi = g % 4;                      // physical 16-byte chunk, group inside it
  const int lc = pc ^ ((r >> 1) & 3);                    // logical chunk stored at this physical position
  const int mt = (int)(tile / kb_total), kb = (int)(tile % kb_total);
  const int row = mt * 128 + r;
  const int col = kb * 64 + lc * 16 + gi * 4;
  uint8_t b[4] = {0, 0, 0, 0};
  if (row < N)
    for (int i = 0; i < 4; ++i)
      if (col + i < K) b[i] = w[(size_t)row * K + col + i];
  const uint32_t v = (uint32_t)b[0] | ((uint32_t)b[2] << 8) | ((uint32_t)b[1] << 16) | ((uint32_t)b[3] << 24);
  reinterpret_cast<uint32_t*>(out)[gid] = v;
}

__global__ void bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __bfloat162float(in[i]);
}

// Inverse of the FP8 packing, with the block-128 scales applied: one thread per 16-byte physical chunk of a
// [128 x 64] tile -> 16 consecutive bf16 of the row-major [N, K] matrix.
__global__ void unpack_fp8_bf16_kernel(const uint8_t* __restrict__ packed, const float* __restrict__ scales,
                                       __nv_bfloat16* __restrict__ out, int N, int K, int kb_total, int ksb, int half_tiles) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;      // (tile, row, physical chunk)
  const size_t total = (size_t)((N + 127) / 128) * kb_total * 128 * 4;
  if (i >= total) return;
  const int p = (int)(i & 3), r = (int)((i >> 2) & 127);
  const size_t tile = i >> 9;
  const int kb = (int)(tile % kb_total), mt = (int)(tile / kb_total);
  const int n = mt * 128 + r;
  const int c = p ^ ((r >> 1) & 3);                                       // logical chunk held by physical chunk p
  const int k0 = kb * 64 + c * 16;
  if (n >= N || k0 >= K) return;
  const uint4 u = *reinterpret_cast<const uint4*>(packed + i * 16);
  const float sc = scales[(size_t)mt * ksb + (k0 >> 7)];
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
  __nv_bfloat16 vals[16];
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    // stored byte order (w0, w2, w1, w3)
    const __nv_fp8_storage_t b0 = (__nv_fp8_storage_t)(w[q] & 0xFF), b2 = (__nv_fp8_storage_t)((w[q] >> 8) & 0xFF);
    const __nv_fp8_storage_t b1 = (__nv_fp8_storage_t)((w[q] >> 16) & 0xFF), b3 = (__nv_fp8_storage_t)(w[q] >> 24);
    const __nv_fp8_storage_t order[4] = {b0, b1, b2, b3};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const __half_raw hr = __nv_cvt_fp8_to_halfraw(order[e], __NV_E4M3);
      vals[q * 4 + e] = __float2bfloat16(__half2float(*reinterpret_cast<const __half*>(&hr)) * sc);
    }
  }
  // half_tiles > 0: the matrix is [gate rows | up rows] of half_tiles 128-row tiles each; the copy interleaves them
  // tile by tile (gate tile j, up tile j, gate tile j+1 ...), so a 256-row GEMM tile holds both halves of 128 features
  const size_t n_out = half_tiles > 0 ? (size_t)(mt < half_tiles ? 2 * mt : 2 * (mt - half_tiles) + 1) * 128 + r : (size_t)n;
  __nv_bfloat16* dst = out + n_out * K + k0;
  if (k0 + 16 <= K && (K & 7) == 0) {
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vals);
    *reinterpret_cast<uint4*>(dst + 8) = *reinterpret_cast<const uint4*>(vals + 8);
  } else {
    for (int e = 0; e < 16 && k0 + e < K; ++e) dst[e] = vals[e];
  }
}

}  // namespace

extern "C" {

// Packed FP8 block-128 weights (b200_prepack_fp8 layout) + fp32 scales [ceil(N/128), ceil(K/128)] -> bf16 [N, K].
static int unpack_fp8_bf16_launch(const void* packed, const float* scales, void* out_bf16, int N, int K, int half_tiles,
                                  cudaStream_t stream) {
  if (N <= 0 || K <= 0 || !packed || !scales || !out_bf16) return -6;
  const int kb_total = (K + 63) / 64;
  const size_t total = (size_t)((N + 127) / 128) * kb_total * 128 * 4;
  unpack_fp8_bf16_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const uint8_t*>(packed), scales, reinterpret_cast<__nv_bfloat16*>(out_bf16), N, K, kb_total, (K + 127) / 128,
      half_tiles);
  return (int)cudaGetLastError();
}

int b200_unpack_fp8_bf16(const void* packed, const float* scales, void* out_bf16, int N, int K, cudaStream_t stream) {
  return unpack_fp8_bf16_launch(packed, scales, out_bf16, N, K, 0, stream);
}

// The same expansion for a [gate | up] matrix of N = 2 I rows (I a multiple of 128): output rows are interleaved in
// 128-row tiles (gate tile 0, up tile 0, gate tile 1, ...), the layout the SwiGLU epilogue of the pair GEMM reads.
int b200_unpack_fp8_bf16_gate_up(const void* packed, const float* scales, void* out_bf16, int N, int K, cudaStream_t stream) {
  if (N <= 0 || N % 256) return -6;
  return unpack_fp8_bf16_launch(packed, scales, out_bf16, N, K, N / 256, stream);
}

unsigned long long b200_prepack_fp8_bytes(int N, int K) {
  return (unsigned long long)((N + 127) / 128) * ((K + 63) / 64) * 8192ull;
}

int b200_prepack_fp8(const void* w_fp8, void* out, int N, int K, cudaStream_t stream) {
  if (N <= 0 || K <= 0) return -6;
  const int kb_total = (K + 63) / 64;
  const size_t total = (size_t)((N + 127) / 128) * kb_total * 128 * 16;
  prepack_fp8_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const uint8_t*>(w_fp8),
                                                                       reinterpret_cast<uint8_t*>(out), N, K, kb_total);
  return (int)cudaGetLastError();
}

int b200_bf16_to_f32(const void* in, float* out, long long n, cudaStream_t stream) {
  if (n <= 0) return -6;
  bf16_to_f32_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(in), out, (size_t)n);
  return (int)cudaGetLastError();
}

}  // extern "C"
