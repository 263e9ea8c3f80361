// Tensor-parallel communicator of the native engine: one NCCL communicator per process, bootstrapped through a file.
// Rank 0 creates the NCCL unique id and writes it (atomically, via rename) to `id_path`; the other ranks poll for the
// file; everyone then calls ncclCommInitRank.  All collectives are enqueued on a caller-supplied stream.
// (Role of cpp_engine/include/tp_comm.hpp:23-75 and cpp_engine/backends/cuda/collective/tp_comm.cpp:49-198, 423-510.)
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <string>
#include <vector>

namespace pocket {

class TpComm {
 public:
  TpComm() = default;
  ~TpComm();
  TpComm(const TpComm&) = delete;
  TpComm& operator=(const TpComm&) = delete;

  // wait_attempts x wait_ms bounds the workers' wait for the id file (default 6000 x 100 ms, as the reference).
  // Throws std::runtime_error with the NCCL / file error.  world == 1 is a no-op communicator.
  void init(int world, int rank, int device, const std::string& id_path, int wait_attempts = 6000, int wait_ms = 100);
  void destroy();
  int world() const { return world_; }
  int rank() const { return rank_; }
  bool active() const { return world_ > 1; }

  void all_reduce_bf16(void* buf, size_t count, cudaStream_t stream);          // in place, sum
  void all_reduce_f32(float* buf, size_t count, cudaStream_t stream);
  void all_gather_bytes(const void* send, void* recv, size_t bytes_per_rank, cudaStream_t stream);
  void broadcast_i32(int32_t* buf, size_t count, int root, cudaStream_t stream);
  // Global arg-max from per-rank winners over vocabulary shards: `val` / `idx` are device arrays of `rows` entries
  // (idx already global ids); `gather` is device scratch of world * rows * 8 bytes.  Returns the winning ids on the
  // host (ties go to the lower id); synchronises the stream.
  std::vector<int32_t> argmax_merge(const float* val, const int32_t* idx, int rows, void* gather, cudaStream_t stream);

 private:
  int world_ = 1, rank_ = 0;
  void* comm_ = nullptr;    // ncclComm_t
};

}  // namespace pocket
