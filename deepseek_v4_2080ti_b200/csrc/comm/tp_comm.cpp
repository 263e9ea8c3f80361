#include "tp_comm.hpp"

#include <nccl.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <thread>

namespace pocket {

namespace {
void nccl_check(ncclResult_t r, const char* what) {
  if (r != ncclSuccess) throw std::runtime_error(std::string(what) + ": " + ncclGetErrorString(r));
}
void cu_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
}  // namespace

TpComm::~TpComm() { destroy(); }

void TpComm::destroy() {
  if (comm_) {
    ncclCommDestroy(reinterpret_cast<ncclComm_t>(comm_));
    comm_ = nullptr;
  }
  world_ = 1;
  rank_ = 0;
}

void TpComm::init(int world, int rank, int device, const std::string& id_path, int wait_attempts, int wait_ms) {
  destroy();
  if (world <= 1) return;
  if (rank < 0 || rank >= world) throw std::runtime_error("tp_comm: rank outside the group");
  if (id_path.empty()) throw std::runtime_error("tp_comm: a multi-rank group needs --nccl-id-path");
  cu_check(cudaSetDevice(device), "cudaSetDevice");
  ncclUniqueId id;
  static_assert(sizeof(id) == NCCL_UNIQUE_ID_BYTES, "unique id size");
  if (rank == 0) {
    nccl_check(ncclGetUniqueId(&id), "ncclGetUniqueId");
    const std::string tmp = id_path + ".tmp." + std::to_string(::getpid());
    {
      std::ofstream f(tmp, std::ios::binary | std::ios::trunc);
      f.write(reinterpret_cast<const char*>(&id), sizeof(id));
      if (!f) throw std::runtime_error("tp_comm: cannot write " + tmp);
    }
    if (std::rename(tmp.c_str(), id_path.c_str()) != 0) throw std::runtime_error("tp_comm: cannot publish " + id_path);
  } else {
    bool ok = false;
    for (int a = 0; a < wait_attempts && !ok; ++a) {
      std::ifstream f(id_path, std::ios::binary);
      if (f) {
        f.read(reinterpret_cast<char*>(&id), sizeof(id));
        ok = f.gcount() == std::streamsize(sizeof(id));
      }
      if (!ok) std::this_thread::sleep_for(std::chrono::milliseconds(wait_ms));
    }
    if (!ok) throw std::runtime_error("tp_comm: timed out waiting for the NCCL id at " + id_path);
  }
  ncclComm_t c = nullptr;
  nccl_check(ncclCommInitRank(&c, world, id, rank), "ncclCommInitRank");
  comm_ = c;
  world_ = world;
  rank_ = rank;
}

void TpComm::all_reduce_bf16(void* buf, size_t count, cudaStream_t stream) {
  if (!active() || count == 0) return;
  nccl_check(ncclAllReduce(buf, buf, count, ncclBfloat16, ncclSum, reinterpret_cast<ncclComm_t>(comm_), stream),
             "ncclAllReduce(bf16)");
}

void TpComm::all_reduce_f32(float* buf, size_t count, cudaStream_t stream) {
  if (!active() || count == 0) return;
  nccl_check(ncclAllReduce(buf, buf, count, ncclFloat32, ncclSum, reinterpret_cast<ncclComm_t>(comm_), stream),
             "ncclAllReduce(f32)");
}

void TpComm::all_gather_bytes(const void* send, void* recv, size_t bytes_per_rank, cudaStream_t stream) {
  if (!active()) {
    if (send != recv) cu_check(cudaMemcpyAsync(recv, send, bytes_per_rank, cudaMemcpyDeviceToDevice, stream), "copy");
    return;
  }
  nccl_check(ncclAllGather(send, recv, bytes_per_rank, ncclUint8, reinterpret_cast<ncclComm_t>(comm_), stream),
             "ncclAllGather");
}

void TpComm::broadcast_i32(int32_t* buf, size_t count, int root, cudaStream_t stream) {
  if (!active() || count == 0) return;
  nccl_check(ncclBroadcast(buf, buf, count, ncclInt32, root, reinterpret_cast<ncclComm_t>(comm_), stream), "ncclBroadcast");
}

std::vector<int32_t> TpComm::argmax_merge(const float* val, const int32_t* idx, int rows, void* gather, cudaStream_t stream) {
  // each rank contributes rows x (value, id); everyone gathers world x rows x 8 bytes and picks the winner on the host
  std::vector<int32_t> out(rows);
  const size_t per = size_t(rows) * 4;
  uint8_t* g = reinterpret_cast<uint8_t*>(gather);
  uint8_t* vals = g;                                   // [world][rows] float
  uint8_t* ids = g + size_t(world_) * per;             // [world][rows] int32
  all_gather_bytes(val, vals, per, stream);
  all_gather_bytes(idx, ids, per, stream);
  std::vector<float> hv(size_t(world_) * rows);
  std::vector<int32_t> hi(size_t(world_) * rows);
  cu_check(cudaMemcpyAsync(hv.data(), vals, hv.size() * 4, cudaMemcpyDeviceToHost, stream), "argmax values");
  cu_check(cudaMemcpyAsync(hi.data(), ids, hi.size() * 4, cudaMemcpyDeviceToHost, stream), "argmax ids");
  cu_check(cudaStreamSynchronize(stream), "argmax merge");
  for (int r = 0; r < rows; ++r) {
    float best = hv[r];
    int32_t bi = hi[r];
    for (int w = 1; w < world_; ++w) {
      const float v = hv[size_t(w) * rows + r];
      const int32_t k = hi[size_t(w) * rows + r];
      if (v > best || (v == best && k < bi)) { best = v; bi = k; }
    }
    out[r] = bi;
  }
  return out;
}

}  // namespace pocket
