// Sequence-parallel residual stream over the peer-memory communicator (comm.h): the reduce + norm + all-gather kernel
// that sits between a row-parallel GEMM in reduce-scatter mode (b200_gemm_wdec_rs) and the next column-parallel GEMM
// in all-gather mode (b200_gemm_wdec_ag).
#pragma once
#include "comm.h"

#define B200_SP_FLAG_ROWS 8   // rows per CTA of the gather kernel = rows per readiness flag of the gathered buffer

#ifdef __cplusplus
extern "C" {
#endif

// h_shard: this rank's rows [rank*rows, (rank+1)*rows) of the residual stream, bf16 [rows, H], local memory.
// with_partials != 0: the previous kernel on every rank's stream was b200_gemm_wdec_rs with token tile rs_bn and
//   N == H; its partials are summed in rank order (rounded to bf16 as an all-reduce would) and added to h_shard.
// gamma != null: the rows are RMS-normalised (weight gamma, or 1 + gamma with unit_offset) and stored into result
//   buffer x_index of every rank (gather != 0) or of this rank only (gather == 0) at row offset rank*rows;
//   with gather != 0 one flag per B200_SP_FLAG_ROWS rows is raised on every peer.
// epoch_word >= 0 (0..3, with gather == 0): the call's epoch is left in a control word for b200_sp_push_rows, which
//   then performs the gather from another stream while the next GEMM already runs on this rank's own rows.
// rows % 8 == 0, H % 8 == 0, world*rows*H <= slot_elems.  Advances the communicator's epoch.
int b200_sp_reduce_norm_gather(const B200Comm* c, void* h_shard, const void* gamma, float eps, int unit_offset,
                               int rows, int H, int with_partials, int rs_bn, int x_index, int gather, int epoch_word,
                               int* status, unsigned long long budget_ns, cudaStream_t stream);

// Deferred all-gather: pushes this rank's rows of gathered buffer x_index to every peer and raises their flags with
// the epoch b200_sp_reduce_norm_gather(..., gather = 0, epoch_word) recorded.  The caller orders it after that call
// (an event) and must not start the next b200_sp_reduce_norm_gather before it has finished.
int b200_sp_push_rows(const B200Comm* c, int rows, int H, int x_index, int epoch_word, cudaStream_t stream);

// Blocks the stream until every peer's rows of the last gather have arrived in this rank's buffer (bounded wait).
// Needed only before kernels that read the gathered buffer without the per-tile wait of b200_gemm_wdec_ag.
int b200_sp_wait_gather(const B200Comm* c, int rows, int* status, unsigned long long budget_ns, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
