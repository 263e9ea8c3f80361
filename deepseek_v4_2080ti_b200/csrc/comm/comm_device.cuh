// Device-side addressing of the symmetric buffer and the epoch hand-over shared by the peer-memory kernels.
#pragma once
#include <cuda_bf16.h>

#include "../ptx/sm100.cuh"
#include "comm.h"

namespace b200 {

__device__ __forceinline__ uint32_t* flag_slot(uint32_t* base, int parity, int src) {
  return base + ((size_t)parity * B200_MAX_RANKS + src) * B200_FLAGS_PER_SLOT;
}
__device__ __forceinline__ __nv_bfloat16* data_slot(void* base, int parity, int src, size_t slot_elems) {
  return reinterpret_cast<__nv_bfloat16*>(base) + ((size_t)parity * B200_MAX_RANKS + src) * slot_elems;
}

// Last CTA to leave publishes the new epoch. All CTAs read the old epoch at entry, before any can leave.
__device__ __forceinline__ void finish_epoch(uint32_t* ctrl, uint32_t epoch) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(&ctrl[1], 1u) + 1;
    if (done == gridDim.x) {
      ctrl[1] = 0;
      __threadfence();
      atomicExch(&ctrl[0], epoch);
    }
  }
}

__device__ __forceinline__ __nv_bfloat16* result_half(void* base, int parity, size_t slot_elems) {
  return reinterpret_cast<__nv_bfloat16*>(base) + (size_t)parity * slot_elems;
}

}  // namespace b200
