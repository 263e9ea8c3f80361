// Symmetric-buffer management and the small stand-alone peer-memory collectives
// (one-shot all-reduce for decode-size payloads, packed arg-max merge).
// The reference's counterpart is its CUDA-IPC one-shot all-reduce, fixed at 4 ranks
// (src/csrc/cuda_kernel_impl.cu:4788-5110) and the packed-u64 max merge over NCCL
// (cpp_engine/backends/cuda/collective/tp_comm.cpp:162-183, 345-364).
#include <cuda_bf16.h>
#include <string.h>

#include "../ptx/sm100.cuh"
#include "comm.h"
#include "comm_device.cuh"

using namespace b200;

namespace {

constexpr size_t kFlagWords = 2ull * B200_MAX_RANKS * B200_FLAGS_PER_SLOT;

// grid = CH chunks; chunk c covers elements [c*per, (c+1)*per). 16-byte vectors.
__global__ void __launch_bounds__(256)
allreduce_oneshot_kernel(B200Comm c, __nv_bfloat16* buf, size_t n, size_t per, int* status, uint64_t budget_ns) {
  const uint32_t epoch = c.ctrl[0] + 1;
  const int parity = epoch & 1;
  const size_t lo = (size_t)blockIdx.x * per;
  const size_t hi = min(n, lo + per);
  // 1. push my chunk to every peer's slot for source = me
  for (int r = 0; r < c.world; ++r) {
    if (r == c.rank) continue;
    __nv_bfloat16* dst = data_slot(c.data[r], parity, c.rank, c.slot_elems);
    for (size_t i = lo + (size_t)threadIdx.x * 8; i < hi; i += 256 * 8) {
      if (i + 8 <= hi) *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(buf + i);
      else for (size_t j = i; j < hi; ++j) dst[j] = buf[j];
    }
  }
  __threadfence_system();
  __syncthreads();
  // 2. raise my flag for this chunk on every peer, then wait for theirs
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < c.world && threadIdx.x != c.rank) {
    const int r = threadIdx.x;
    st_release_sys(flag_slot(c.flags[r], parity, c.rank) + blockIdx.x, epoch);
    if (!wait_flag_ge(flag_slot(c.flags[c.rank], parity, r) + blockIdx.x, epoch, budget_ns)) {
      atomicExch(status, ERR_WAIT_PEER);
      failed = 1;
    }
  }
  __syncthreads();
  // 3. reduce (rank order is the same everywhere: results are bit-identical across ranks)
  if (!failed) {
    for (size_t i = lo + (size_t)threadIdx.x * 8; i < hi; i += 256 * 8) {
      const int cnt = (int)min((size_t)8, hi - i);
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int r = 0; r < c.world; ++r) {
        const __nv_bfloat16* src = (r == c.rank) ? buf : data_slot(c.data[c.rank], parity, r, c.slot_elems);
        if (cnt == 8) {
          const uint4 u = *reinterpret_cast<const uint4*>(src + i);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const float2 f = __bfloat1622float2(h[k]);
            acc[2 * k] += f.x;
            acc[2 * k + 1] += f.y;
          }
        } else {
          for (int k = 0; k < cnt; ++k) acc[k] += __bfloat162float(src[i + k]);
        }
      }
      // own values are read before being overwritten: each element is owned by exactly one thread
      if (cnt == 8) {
        uint4 u;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
        *reinterpret_cast<uint4*>(buf + i) = u;
      } else {
        for (int k = 0; k < cnt; ++k) buf[i + k] = __float2bfloat16(acc[k]);
      }
    }
  }
  finish_epoch(c.ctrl, epoch);
}

// One CTA. Rows <= 1024. Each rank pushes (value, index) per row into the peers' data slots (8 bytes/row).
__global__ void __launch_bounds__(256)
argmax_merge_kernel(B200Comm c, const float* val, const int* idx, int rows, int* out_idx, int* status,
                    uint64_t budget_ns) {
  const uint32_t epoch = c.ctrl[0] + 1;
  const int parity = epoch & 1;
  for (int r = 0; r < c.world; ++r) {
    if (r == c.rank) continue;
    uint2* dst = reinterpret_cast<uint2*>(data_slot(c.data[r], parity, c.rank, c.slot_elems));
    for (int i = threadIdx.x; i < rows; i += blockDim.x) dst[i] = make_uint2(__float_as_uint(val[i]), (uint32_t)idx[i]);
  }
  __threadfence_system();
  __syncthreads();
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (threadIdx.x < c.world && threadIdx.x != c.rank) {
    const int r = threadIdx.x;
    st_release_sys(flag_slot(c.flags[r], parity, c.rank), epoch);
    if (!wait_flag_ge(flag_slot(c.flags[c.rank], parity, r), epoch, budget_ns)) {
      atomicExch(status, ERR_WAIT_PEER);
      failed = 1;
    }
  }
  __syncthreads();
  if (!failed) {
    for (int i = threadIdx.x; i < rows; i += blockDim.x) {
      float best = val[i];
      int bi = idx[i];
      for (int r = 0; r < c.world; ++r) {
        if (r == c.rank) continue;
        const uint2 u = reinterpret_cast<const uint2*>(data_slot(c.data[c.rank], parity, r, c.slot_elems))[i];
        const float v = __uint_as_float(u.x);
        const int k = (int)u.y;
        if (v > best || (v == best && k < bi)) { best = v; bi = k; }
      }
      out_idx[i] = bi;
    }
  }
  finish_epoch(c.ctrl, epoch);
}

}  // namespace

extern "C" {

unsigned long long b200_comm_buffer_bytes(unsigned long long slot_elems) {
  // flags (2 banks) | ctrl (256 B) | data | result (2 buffers)
  return 2 * kFlagWords * 4 + 256 + 2ull * B200_MAX_RANKS * slot_elems * 2 + 2ull * slot_elems * 2;
}

int b200_comm_alloc(unsigned long long bytes, void** out) {
  cudaError_t e = cudaMalloc(out, bytes);
  if (e != cudaSuccess) return (int)e;
  return (int)cudaMemset(*out, 0, bytes);
}
int b200_comm_free(void* p) { return (int)cudaFree(p); }

int b200_comm_ipc_handle(void* p, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) return (int)e;
  static_assert(sizeof(h) == 64, "IPC handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
int b200_comm_ipc_open(const void* handle64, void** out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  return (int)cudaIpcOpenMemHandle(out, h, cudaIpcMemLazyEnablePeerAccess);
}
int b200_comm_ipc_close(void* p) { return (int)cudaIpcCloseMemHandle(p); }

int b200_comm_enable_peer(int peer_device) {
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    cudaGetLastError();
    return 0;
  }
  return (int)e;
}

int b200_comm_init(B200Comm* c, int rank, int world, void* const* bases, unsigned long long slot_elems) {
  if (world < 1 || world > B200_MAX_RANKS || rank < 0 || rank >= world) return -ERR_BAD_ARG;
  memset(c, 0, sizeof(*c));
  c->rank = rank;
  c->world = world;
  c->slot_elems = slot_elems;
  for (int r = 0; r < world; ++r) {
    uint8_t* b = reinterpret_cast<uint8_t*>(bases[r]);
    c->flags[r] = reinterpret_cast<uint32_t*>(b);
    c->flags2[r] = reinterpret_cast<uint32_t*>(b + kFlagWords * 4);
    c->data[r] = b + 2 * kFlagWords * 4 + 256;
    c->result[r] = b + 2 * kFlagWords * 4 + 256 + 2ull * B200_MAX_RANKS * slot_elems * 2;
  }
  c->ctrl = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(bases[rank]) + 2 * kFlagWords * 4);
  return 0;
}

int b200_allreduce_oneshot(const B200Comm* c, void* buf, long long n, int* status, unsigned long long budget_ns,
                           cudaStream_t stream) {
  if (n <= 0 || (unsigned long long)n > c->slot_elems) return -ERR_BAD_ARG;
  if (c->world == 1) return 0;
  if (budget_ns == 0) budget_ns = B200_WAIT_BUDGET_NS;
  // chunks of >= 2048 elements (16 B per thread per pass), at most 128 CTAs and FLAGS_PER_SLOT flags
  size_t chunks = ((size_t)n + 2047) / 2048;
  if (chunks > 128) chunks = 128;
  size_t per = (((size_t)n + chunks - 1) / chunks + 7) / 8 * 8;
  chunks = ((size_t)n + per - 1) / per;
  allreduce_oneshot_kernel<<<(unsigned)chunks, 256, 0, stream>>>(*c, reinterpret_cast<__nv_bfloat16*>(buf), (size_t)n,
                                                                 per, status, budget_ns);
  return (int)cudaGetLastError();
}

int b200_argmax_merge(const B200Comm* c, const float* val, const int* idx, int rows, int* out_idx, int* status,
                      unsigned long long budget_ns, cudaStream_t stream) {
  if (rows <= 0 || (unsigned long long)rows * 4 > c->slot_elems) return -ERR_BAD_ARG;
  if (budget_ns == 0) budget_ns = B200_WAIT_BUDGET_NS;
  argmax_merge_kernel<<<1, 256, 0, stream>>>(*c, val, idx, rows, out_idx, status, budget_ns);
  return (int)cudaGetLastError();
}

}  // extern "C"
