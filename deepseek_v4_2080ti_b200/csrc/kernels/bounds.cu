// Index checks for the debug mode of the op front-ends (B200_BOUNDS_CHECK=1): before a kernel that addresses memory
// through an index tensor (token ids, cache element offsets, page-table entries, state slots, selected key rows) is
// launched, this kernel scans the indices.  An index outside [lo, hi) is recorded in the device error word - code
// ERR_BOUNDS in the low byte, the checked site in the next byte, the position of the offending element above - and
// REPLACED by a safe value, so that the kernel that follows addresses valid memory: the failure is a status the host
// reads, never a fault.  `keep` is a sentinel that is left alone (-1 = "no entry" in the sparse index lists).
// The reference validates index tensors on the host inside its pybind ops (src/csrc/cuda_kernel.cpp TORCH_CHECKs on
// shapes) and has no device-side check; a device memory checker cannot be run where this package is tested.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../ptx/sm100.cuh"

namespace {

__global__ void check_indices_kernel(int* __restrict__ idx, long long n, int lo, int hi, int keep, int has_keep,
                                     int replace, int* __restrict__ status, int site) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const int v = idx[i];
  if ((has_keep && v == keep) || (v >= lo && v < hi)) return;
  idx[i] = replace;
  const int pos = (int)(i > 0xFFFF ? 0xFFFF : i);
  atomicCAS(status, 0, b200::ERR_BOUNDS | ((site & 0xFF) << 8) | (pos << 16));
}

}  // namespace

extern "C" int b200_check_indices(int* idx, long long n, int lo, int hi, int keep, int has_keep, int replace,
                                  int* status, int site, cudaStream_t stream) {
  if (!idx || !status || n < 0 || hi <= lo || replace < lo || replace >= hi) return -b200::ERR_BAD_ARG;
  if (n == 0) return 0;
  check_indices_kernel<<<(unsigned)((n + 255) / 256), 256, 0, stream>>>(idx, n, lo, hi, keep, has_keep, replace, status, site);
  return (int)cudaGetLastError();
}
