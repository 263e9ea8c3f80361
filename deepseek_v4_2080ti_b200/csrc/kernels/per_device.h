// Function attributes (cudaFuncSetAttribute) belong to a device, not to the process: a launcher that sets one
// behind a process-wide flag leaves every other device of a multi-GPU process unconfigured.  PerDeviceOnce keeps
// one flag per device ordinal; slot() returns the flag of the current device.
#pragma once
#include <cuda_runtime.h>

namespace b200 {
struct PerDeviceOnce {
  bool done[64] = {};
  bool& slot() {
    int d = 0;
    cudaGetDevice(&d);
    return done[d & 63];
  }
};
}  // namespace b200
