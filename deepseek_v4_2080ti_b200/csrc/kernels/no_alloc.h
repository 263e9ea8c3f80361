// Split-K GEMM entry point that never allocates.
//
// This entry point has no counterpart in the reference; it exists for hosts that
// embed the kernel library but are not allowed to touch the CUDA allocator at
// the moment they need a GEMM:
//   * an engine that hands all device memory to its own pool at start-up, so a
//     later cudaMalloc would fail or fragment that pool;
//   * a latency-critical serving loop that has promised "no allocator calls after
//     warm-up", because cudaMalloc/cudaFree can take driver-wide locks and
//     synchronise the device;
//   * plain-C or foreign-language callers that reach the library through its C
//     symbols only and have no torch (or other) caching allocator to borrow
//     scratch from.
// The regular entry point (b200_gemm_wdec with splits > 1) needs a caller-provided
// fp32 workspace of splits*T*N floats.  Here that workspace is a fixed array that
// lives inside the library image instead.
//
// Contract
//   * Same math and arguments as b200_gemm_wdec followed by b200_splitk_reduce:
//     out_bf16[T, N] = X[T, K] * W[N, K]^T (+ residual), K split `splits` ways.
//     The caller still owns and passes every input and output buffer and the
//     int32 status word.
//   * Scratch: a file-scope device array of B200_NOALLOC_MAX_FLOATS floats
//     (16 MiB).  Every GPU that loads the library keeps that much memory reserved
//     until the process exits.  splits*T*N above the limit is refused with
//     B200_ERR_SCRATCH_TOO_SMALL and a message on stderr; nothing is launched.
//   * No cudaMalloc, cudaFree, or allocating library routine is called, on the
//     first call or later.
//   * The first call on each device looks up the array's device address (with that
//     device current) and caches it.  Make that first call during start-up, before
//     any stream capture begins on that device.
//   * All calls on one device share the one array, and it keeps whatever the
//     previous call left there.  The kernels overwrite every partial they later
//     read, so nothing has to be cleared between calls; but two calls that overlap
//     in time on the same GPU (different streams, or different host threads) race
//     on the scratch.  Serialise them on one stream.
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_NOALLOC_MAX_FLOATS (4ll * 1024 * 1024)
#define B200_ERR_SCRATCH_TOO_SMALL (-7)

// Largest splits*T*N (in floats) the built-in scratch can hold.
long long b200_gemm_wdec_noalloc_max_floats(void);

// wfmt, W, scales, X, residual, T, N, K, status, stream: as for b200_gemm_wdec.
// Returns 0, a cudaError_t, a negative b200 error code, or B200_ERR_SCRATCH_TOO_SMALL.
int b200_gemm_wdec_splitk_noalloc(int wfmt, const void* W, const float* scales, const void* X,
                                  void* out_bf16, const void* residual, int T, int N, int K,
                                  int splits, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
