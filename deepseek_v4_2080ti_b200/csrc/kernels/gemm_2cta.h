// bf16 GEMM on CTA pairs (tcgen05.mma.cta_group::2), see gemm_bf16_2cta.cu.
#pragma once
#include <cuda_runtime.h>

#include "../comm/comm.h"

#ifdef __cplusplus
extern "C" {
#endif

// Process-wide switch (default on) and the shape test: T % 256 == 0, N % 256 == 0, K % 64 == 0.
void b200_gemm_2cta_enable(int on);
int b200_gemm_2cta_enabled(void);
int b200_gemm_2cta_supported(int T, int N, int K);

// out[T, N] = X[T, K] W[N, K]^T, all bf16 (mode 0); mode 3 pushes the partial tiles to the owners of the token rows
// instead (reduce-scatter half of the sequence-parallel path, comm / sp_rows / n_rot as b200_gemm_wdec_rs computes
// them); ag_wait != 0: X is the gathered activation buffer, a token half-tile is loaded once its flags are up.
int b200_gemm_bf16_2cta(const void* W, const void* X, void* out_bf16, int T, int N, int K, int mode,
                        const B200Comm* comm, int sp_rows, int n_rot, int ag_wait, int ag_flag_rows,
                        unsigned long long budget_ns, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
