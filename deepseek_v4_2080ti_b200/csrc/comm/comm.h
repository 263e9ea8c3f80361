// Peer-memory communication context shared by the fused compute+collective kernels.
//
// Every rank owns one "symmetric" buffer of identical layout and holds a pointer to every
// peer's buffer (CUDA IPC across processes, or plain peer access inside one process).
//   flags  : uint32 [2 banks][2 parities][MAX_RANKS sources][FLAGS_PER_SLOT]   written by peers, read locally
//            (bank 0: "partial tile arrived", bank 1: "reduced tile arrived")
//   ctrl   : uint32 [16]   [0] = epoch of the last finished collective, [1] = CTA exit counter
//   data   : bf16   [2 parities][MAX_RANKS sources][slot_elems]        written by peers, read locally
//   result : bf16   [2 buffers][slot_elems]   reduced outputs of the two-shot GEMM epilogue, written by tile owners
// A collective call number ("epoch") is kept on the device so CUDA-graph replays advance it
// without any host-side argument changing; all ranks issue identical call sequences, so their
// epochs agree.  Parity = epoch & 1 selects the buffer half: a peer can only be one call ahead.
// All waits on peer flags are bounded (sm100.cuh wait_flag_ge) and report ERR_WAIT_PEER.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#define B200_MAX_RANKS 8
#define B200_FLAGS_PER_SLOT 4096
#define B200_CTRL_WORDS 16

struct B200Comm {
  int rank, world;
  unsigned long long slot_elems;        // bf16 elements per (parity, source) data slot
  uint32_t* flags[B200_MAX_RANKS];      // base of rank r's flag region (peer-mapped)
  uint32_t* ctrl;                       // local control words
  void* data[B200_MAX_RANKS];           // base of rank r's data region (peer-mapped)
  uint32_t* flags2[B200_MAX_RANKS];     // second flag bank of rank r
  void* result[B200_MAX_RANKS];         // base of rank r's result region
};

#ifdef __cplusplus
extern "C" {
#endif

// Bytes a symmetric buffer needs for `slot_elems` elements per slot.
unsigned long long b200_comm_buffer_bytes(unsigned long long slot_elems);
// cudaMalloc + zero. The buffer must be allocated with this call so that IPC export works.
int b200_comm_alloc(unsigned long long bytes, void** out);
int b200_comm_free(void* p);
// 64-byte IPC handle of a buffer allocated by b200_comm_alloc; open / close a peer's handle.
int b200_comm_ipc_handle(void* p, void* handle64);
int b200_comm_ipc_open(const void* handle64, void** out);
int b200_comm_ipc_close(void* p);
// Enable peer access from the current device to `peer_device` (single-process multi-GPU use).
int b200_comm_enable_peer(int peer_device);
// Fill a context from the base pointers of all ranks' buffers (bases[rank] is the local one).
int b200_comm_init(B200Comm* c, int rank, int world, void* const* bases, unsigned long long slot_elems);

// Stand-alone one-shot all-reduce (sum) of n bf16 values in place: every rank pushes its vector to
// all peers, waits for theirs, and sums in fp32.  n <= slot_elems.  `status` receives ERR_WAIT_PEER
// if a peer's data did not arrive within the wait budget (budget_ns == 0 selects the default 2 s).
int b200_allreduce_oneshot(const B200Comm* c, void* buf_bf16, long long n, int* status,
                           unsigned long long budget_ns, cudaStream_t stream);
// Arg-max merge: each rank contributes rows of (value, index); all ranks get the winning index per row.
int b200_argmax_merge(const B200Comm* c, const float* val, const int* idx, int rows, int* out_idx, int* status,
                      unsigned long long budget_ns, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
