// Entry points of the weight-decoding GEMM for bf16, FP8 block-128 and FP4 weights (kernel: gemm_wdec_kernel.cuh).
#include "gemm_wdec_kernel.cuh"
#include "gemm_2cta.h"

using namespace b200;

// What a fused compute+collective entry point adds to the plain launch; passed down explicitly so that host
// threads launching GEMMs side by side never see each other's collective.
struct FusedOpts {
  const B200Comm* comm = nullptr;
  int ar_mode = 0;                 // 1 one-shot all-reduce, 2 two-shot, 3 reduce-scatter push
  size_t result_off = 0;
  unsigned long long budget_ns = 0;
  int sp_rows = 0;                 // rows per owner shard (reduce-scatter push, all-gather wait)
  int ag_wait = 0, ag_flag_rows = 0;
  int bn = 0;                      // token tile forced by the collective's layout (0: by T)
  int n_rot = 0;
};
static int gemm_wdec_launch(int wfmt, const void* W, const float* scales, const void* X, void* out_bf16,
                            float* out_f32, const void* residual, int T, int N, int K, int splits,
                            int* tile_counters, int* status, cudaStream_t stream, const FusedOpts* fo);

extern "C" int b200_gemm_pick_bn(int T) {
  if (T <= 16) return 16;
  if (T <= 32) return 32;
  if (T <= 64) return 64;
  if (T <= 128) return 128;
  return 256;
}

// wfmt: 0 = bf16 weights [N, K]; 1 = FP8 E4M3 weights in the tile-major layout
// [ceil(N/128)][ceil(K/64)][128 rows][64 bytes] (zero padded; each 4-byte group stored as
// (w0,w2,w1,w3); the four 16-byte chunks of row r stored at chunk index c ^ ((r >> 1) & 3), which is
// the 64-byte shared-memory swizzle, so that the same bytes can also feed FP8 tensor-core tiles
// directly, see gemm_w8a8s.cu) with fp32 scales [ceil(N/128), ceil(K/128)].
// splits == 1: writes bf16 `out` (adds `residual` when given), or fp32 `out_f32` when out == null.
// splits  > 1: writes fp32 partials to out_f32 [splits, T, N] (caller reduces).
extern "C" int b200_gemm_wdec_ex(int wfmt, const void* W, const float* scales, const void* X,
                                 void* out_bf16, float* out_f32, const void* residual, int T, int N,
                                 int K, int splits, int* tile_counters, int* status, cudaStream_t stream);

extern "C" int b200_gemm_wdec(int wfmt, const void* W, const float* scales, const void* X,
                              void* out_bf16, float* out_f32, const void* residual, int T, int N,
                              int K, int splits, int* status, cudaStream_t stream) {
  return b200_gemm_wdec_ex(wfmt, W, scales, X, out_bf16, out_f32, residual, T, N, K, splits, nullptr, status,
                           stream);
}

// As b200_gemm_wdec, plus the in-kernel split-K fix-up: with splits > 1, out_bf16, out_f32 (scratch
// for splits*T*N floats) and tile_counters (ceil(N/128)*ceil(T/BN) zeroed ints, left zeroed) all set,
// the kernel itself reduces the partials and writes bf16 (+ residual); no second launch is needed.
extern "C" int b200_gemm_wdec_ex(int wfmt, const void* W, const float* scales, const void* X,
                                 void* out_bf16, float* out_f32, const void* residual, int T, int N,
                                 int K, int splits, int* tile_counters, int* status, cudaStream_t stream) {
  return gemm_wdec_launch(wfmt, W, scales, X, out_bf16, out_f32, residual, T, N, K, splits, tile_counters, status,
                          stream, nullptr);
}

static int gemm_wdec_launch(int wfmt, const void* W, const float* scales, const void* X, void* out_bf16,
                            float* out_f32, const void* residual, int T, int N, int K, int splits,
                            int* tile_counters, int* status, cudaStream_t stream, const FusedOpts* fo) {
  if (T <= 0 || N <= 0 || K <= 0 || (K % 16) != 0 || splits < 1) return -ERR_BAD_ARG;
  const int BN = (fo && fo->bn) ? fo->bn : b200_gemm_pick_bn(T);
  {
    // prefill-sized bf16 problems that tile evenly go to the CTA-pair kernel (256 x 256 tiles, gemm_bf16_2cta.cu)
    const int mode = fo ? fo->ar_mode : 0;
    const bool sp_ok = !fo || !fo->comm || (!fo->sp_rows && !fo->ag_wait) || (fo->sp_rows % 256 == 0);
    if (wfmt == WF_BF16 && BN == 256 && splits == 1 && !residual && !out_f32 && (mode == 0 || mode == 3) &&
        (out_bf16 || mode == 3) && sp_ok && b200_gemm_2cta_supported(T, N, K)) {
      // the rotation was computed in units of this launcher's token tile, which is also 256 here
      return b200_gemm_bf16_2cta(W, X, out_bf16, T, N, K, mode, fo ? fo->comm : nullptr, fo ? fo->sp_rows : 0,
                                 fo ? fo->n_rot : 0, fo ? fo->ag_wait : 0, fo ? fo->ag_flag_rows : 0,
                                 fo ? fo->budget_ns : 0, status, stream);
    }
  }
  GemmParams p;
  p.T = T; p.N = N; p.K = K;
  p.m_tiles = (N + BM - 1) / BM;
  p.n_tiles = (T + BN - 1) / BN;
  p.kb_total = (K + BK - 1) / BK;
  if (splits > p.kb_total) splits = p.kb_total;
  {
    // no split may end up with an empty K range (its accumulator would never be written)
    const int per = (p.kb_total + splits - 1) / splits;
    splits = (p.kb_total + per - 1) / per;
  }
  p.splits = splits;
  p.scales = scales;
  p.scale_ld = (K + 127) / 128;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.out_f32 = out_f32;
  p.residual = reinterpret_cast<const __nv_bfloat16*>(residual);
  p.ldo = N;
  p.status = status;
  p.tile_counters = tile_counters;
  p.work_table = nullptr;
  p.num_work = nullptr;
  p.w_group_stride = 0;
  p.scale_group_stride = 0;
  if (splits > 1 && out_bf16 && !tile_counters) return -ERR_BAD_ARG;
  p.ar_mode = 0;
  p.ar_budget_ns = 0;
  p.result_off = 0;
  p.n_rot = 0;
  p.sp_rows = 0;
  p.ag_wait = 0;
  p.ag_flag_rows = 0;
  p.lut = nullptr;
  memset(&p.comm, 0, sizeof(p.comm));
  if (fo && fo->comm) {
    if (splits != 1 || (!out_bf16 && fo->ar_mode != 3)) return -ERR_BAD_ARG;
    p.ar_mode = fo->ar_mode;
    p.ar_budget_ns = fo->budget_ns;
    p.comm = *fo->comm;
    p.result_off = fo->result_off;
    p.n_rot = fo->n_rot;
    p.sp_rows = fo->sp_rows;
    p.ag_wait = fo->ag_wait;
    p.ag_flag_rows = fo->ag_flag_rows;
  }
  if ((splits > 1 || !out_bf16) && !out_f32 && p.ar_mode != 3) return -ERR_BAD_ARG;
  if (wfmt == WF_FP8_B128) {
    // the decode warps keep at most 256 block scales (K range of 32768) per tile in registers
    const int per = (p.kb_total + splits - 1) / splits;
    if (per / 2 + 2 > 256) return -ERR_BAD_ARG;
  }
  if (wfmt == WF_FP4 && (K % 64) != 0) return -ERR_BAD_ARG;

  CUtensorMap tmW, tmX;
  bool ok = make_tmap_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, T, K, (uint64_t)K * 2, BN, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  p.w_tiled = nullptr;
  if (wfmt == WF_BF16) {
    ok = ok && make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, N, K, (uint64_t)K * 2, BM, BK,
                            CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    p.w_tiled = reinterpret_cast<const uint8_t*>(W);   // fetched with untiled bulk copies, no tensor map
    tmW = tmX;
  }
  if (!ok) return -ERR_BAD_ARG;

#define B200_DISPATCH(BN_)                                                             \
  case BN_:                                                                            \
    return wfmt == WF_BF16       ? launch_one<BN_, WF_BF16>(tmW, tmX, p, stream)       \
           : wfmt == WF_FP8_B128 ? launch_one<BN_, WF_FP8_B128>(tmW, tmX, p, stream)   \
           : wfmt == WF_FP4      ? launch_one<BN_, WF_FP4>(tmW, tmX, p, stream)        \
                                 : -ERR_BAD_ARG;
  switch (BN) {
    B200_DISPATCH(16)
    B200_DISPATCH(32)
    B200_DISPATCH(64)
    B200_DISPATCH(128)
    B200_DISPATCH(256)
  }
#undef B200_DISPATCH
  return -ERR_BAD_ARG;
}

// Grouped GEMM over ragged row segments (routed experts): out[r, :] = X[r, :] * W_g^T for every row r of the
// segment the device-side work table assigns to group g.  X / out: [rows_total, K] / [rows_total, N] bf16 with the
// rows of one group contiguous; W: `groups` matrices of N x K back to back (tile-major packed for FP8 / FP4, plain
// [groups * N, K] for bf16, N % 128 == 0); scales (FP8): [groups][ceil(N/128)][K/128] fp32.
// work_table / num_work are produced on the device (b200_moe_build_work); bn is the token tile (16..256) the
// table was built for.  No host synchronisation is needed between routing and this call.
extern "C" int b200_gemm_wdec_grouped(int wfmt, const void* W, const float* scales, const void* X, void* out_bf16,
                                      int rows_total, int N, int K, int groups, const void* work_table,
                                      const int* num_work, int bn, int* status, cudaStream_t stream) {
  if (rows_total <= 0 || N <= 0 || K <= 0 || (K % 16) != 0 || groups <= 0 || !work_table || !num_work || !out_bf16)
    return -ERR_BAD_ARG;
  if (bn != 16 && bn != 32 && bn != 64 && bn != 128 && bn != 256) return -ERR_BAD_ARG;
  if (wfmt == WF_BF16 && (N % BM) != 0) return -ERR_BAD_ARG;
  if (wfmt == WF_FP4 && (K % 64) != 0) return -ERR_BAD_ARG;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.T = rows_total; p.N = N; p.K = K;
  p.m_tiles = (N + BM - 1) / BM;
  p.n_tiles = 1;
  p.kb_total = (K + BK - 1) / BK;
  p.splits = 1;
  p.scales = scales;
  p.scale_ld = (K + 127) / 128;
  p.out = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  p.ldo = N;
  p.status = status;
  p.work_table = reinterpret_cast<const int4*>(work_table);
  p.num_work = num_work;
  p.w_group_stride = (size_t)p.m_tiles * p.kb_total * raw_stage_bytes(wfmt);
  p.scale_group_stride = (size_t)p.m_tiles * p.scale_ld;
  if (wfmt == WF_FP8_B128 && p.kb_total / 2 + 2 > 256) return -ERR_BAD_ARG;
  CUtensorMap tmW, tmX;
  bool ok = make_tmap_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, X, rows_total, K, (uint64_t)K * 2, bn, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (wfmt == WF_BF16) {
    ok = ok && make_tmap_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, W, (uint64_t)groups * N, K, (uint64_t)K * 2, BM,
                            BK, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    p.w_tiled = reinterpret_cast<const uint8_t*>(W);
    tmW = tmX;
  }
  if (!ok) return -ERR_BAD_ARG;
#define B200_DISPATCH_G(BN_)                                                           \
  case BN_:                                                                            \
    return wfmt == WF_BF16       ? launch_one<BN_, WF_BF16>(tmW, tmX, p, stream)       \
           : wfmt == WF_FP8_B128 ? launch_one<BN_, WF_FP8_B128>(tmW, tmX, p, stream)   \
           : wfmt == WF_FP4      ? launch_one<BN_, WF_FP4>(tmW, tmX, p, stream)        \
                                 : -ERR_BAD_ARG;
  switch (bn) {
    B200_DISPATCH_G(16)
    B200_DISPATCH_G(32)
    B200_DISPATCH_G(64)
    B200_DISPATCH_G(128)
    B200_DISPATCH_G(256)
  }
#undef B200_DISPATCH_G
  return -ERR_BAD_ARG;
}

// Row-parallel GEMM fused with a one-shot all-reduce over peer memory: every rank calls this with its
// K-shard of W and X; all ranks end with out = sum_r X_r W_r^T (+ residual). T*N <= comm->slot_elems and
// ceil(N/128) * ceil(T/BN) <= B200_FLAGS_PER_SLOT. With world == 1 this is the plain GEMM.
extern "C" int b200_gemm_wdec_allreduce(int wfmt, const void* W, const float* scales, const void* X,
                                        void* out_bf16, const void* residual, int T, int N, int K,
                                        const B200Comm* comm, unsigned long long budget_ns, int* status,
                                        cudaStream_t stream) {
  if (!comm || comm->world <= 1)
    return b200_gemm_wdec(wfmt, W, scales, X, out_bf16, nullptr, residual, T, N, K, 1, status, stream);
  if ((unsigned long long)T * N > comm->slot_elems || (N % 8) != 0) return -ERR_BAD_ARG;
  const int BN = b200_gemm_pick_bn(T);
  if ((long long)((N + BM - 1) / BM) * ((T + BN - 1) / BN) > B200_FLAGS_PER_SLOT) return -ERR_BAD_ARG;
  FusedOpts fo;
  fo.comm = comm;
  fo.ar_mode = 1;
  fo.budget_ns = budget_ns ? budget_ns : B200_WAIT_BUDGET_NS;
  return gemm_wdec_launch(wfmt, W, scales, X, out_bf16, nullptr, residual, T, N, K, 1, nullptr, status, stream, &fo);
}

// Two-shot variant: tile w is reduced by rank w % world and the reduced tile is pushed into every rank's result
// region; the output of this call is comm->result[rank] + result_index * slot_elems (bf16 [T, N]), valid until the
// call after next that uses the same result_index.  result_index is 0 or 1.
extern "C" int b200_gemm_wdec_allreduce2(int wfmt, const void* W, const float* scales, const void* X,
                                         const void* residual, int T, int N, int K, const B200Comm* comm,
                                         int result_index, unsigned long long budget_ns, int* status,
                                         cudaStream_t stream) {
  if (!comm || comm->world <= 1 || result_index < 0 || result_index > 1) return -ERR_BAD_ARG;
  if ((unsigned long long)T * N > comm->slot_elems || (N % 8) != 0) return -ERR_BAD_ARG;
  const int BN = b200_gemm_pick_bn(T);
  if ((long long)((N + BM - 1) / BM) * ((T + BN - 1) / BN) > B200_FLAGS_PER_SLOT) return -ERR_BAD_ARG;
  FusedOpts fo;
  fo.comm = comm;
  fo.ar_mode = 2;
  fo.budget_ns = budget_ns ? budget_ns : B200_WAIT_BUDGET_NS;
  fo.result_off = (size_t)result_index * comm->slot_elems;
  void* out = reinterpret_cast<__nv_bfloat16*>(comm->result[comm->rank]) + fo.result_off;
  return gemm_wdec_launch(wfmt, W, scales, X, out, nullptr, residual, T, N, K, 1, nullptr, status, stream, &fo);
}

// Token tile of the sequence-parallel GEMMs for a shard of `sp_rows` rows: the largest tile that divides the shard
// and whose kernel instance carries the epilogue staging (0 = this shape cannot run sequence-parallel).
extern "C" int b200_gemm_sp_bn(int wfmt, int sp_rows) {
  if (wfmt == WF_BF16 && sp_rows % 256 == 0) return 256;
  if ((wfmt == WF_BF16 || wfmt == WF_FP8_B128) && sp_rows % 128 == 0) return 128;
  return 0;
}

// Row-parallel GEMM whose epilogue is the push half of a reduce-scatter (ar_mode 3 in gemm_wdec_kernel.cuh): the
// T = world * sp_rows token rows are owned in contiguous shards; every partial tile goes only to its owner's slot
// for source = this rank, with one flag per tile.  There is no local output: the owner's
// b200_sp_reduce_norm_gather (comm/sp_comm.cu) sums the partials.  Returns the token tile used in *bn_out.
extern "C" int b200_gemm_wdec_rs(int wfmt, const void* W, const float* scales, const void* X, int T, int N, int K,
                                 const B200Comm* comm, unsigned long long budget_ns, int* bn_out, int* status,
                                 cudaStream_t stream) {
  if (!comm || comm->world <= 1 || T % comm->world || (N % 8) != 0) return -ERR_BAD_ARG;
  const int sp_rows = T / comm->world;
  const int bn = b200_gemm_sp_bn(wfmt, sp_rows);
  if (!bn) return -ERR_BAD_ARG;
  if ((unsigned long long)sp_rows * N > comm->slot_elems) return -ERR_BAD_ARG;
  if ((long long)((N + BM - 1) / BM) * (sp_rows / bn) > B200_FLAGS_PER_SLOT) return -ERR_BAD_ARG;
  FusedOpts fo;
  fo.comm = comm;
  fo.ar_mode = 3;
  fo.budget_ns = budget_ns ? budget_ns : B200_WAIT_BUDGET_NS;
  fo.sp_rows = sp_rows;
  fo.bn = bn;
  fo.n_rot = ((comm->rank + 1) % comm->world) * (sp_rows / bn);   // start with the next rank's shard, own shard last
  // the CTA-pair kernel (taken by the launcher for evenly tiling bf16 problems) raises its flags per 128-row block
  const bool pair = wfmt == WF_BF16 && bn == 256 && b200_gemm_2cta_supported(T, N, K);
  if (bn_out) *bn_out = pair ? 128 : bn;
  return gemm_wdec_launch(wfmt, W, scales, X, nullptr, nullptr, nullptr, T, N, K, 1, nullptr, status, stream, &fo);
}

// Column-parallel GEMM on activations that the peers gather into this rank's memory (all-gather + GEMM): X is the
// local [T, K] buffer that b200_sp_reduce_norm_gather fills on every rank; rows of shard s != rank become valid when
// rank s raises their flags (one per flag_rows rows), and the producer warp waits for a tile's flags before loading
// it.  Token tiles are visited own shard first.  Everything else as b200_gemm_wdec with splits == 1.
extern "C" int b200_gemm_wdec_ag(int wfmt, const void* W, const float* scales, const void* X, void* out_bf16, int T,
                                 int N, int K, const B200Comm* comm, int flag_rows, unsigned long long budget_ns,
                                 int* status, cudaStream_t stream) {
  if (!comm || comm->world <= 1 || T % comm->world || flag_rows <= 0 || !out_bf16) return -ERR_BAD_ARG;
  const int sp_rows = T / comm->world;
  int bn = b200_gemm_pick_bn(T);
  while (bn > 16 && sp_rows % bn) bn >>= 1;     // a token tile must not straddle two owners
  if (sp_rows % bn || sp_rows % flag_rows || sp_rows / flag_rows > B200_FLAGS_PER_SLOT) return -ERR_BAD_ARG;
  FusedOpts fo;
  fo.comm = comm;
  fo.ar_mode = 0;
  fo.budget_ns = budget_ns ? budget_ns : B200_WAIT_BUDGET_NS;
  fo.sp_rows = sp_rows;
  fo.ag_wait = 1;
  fo.ag_flag_rows = flag_rows;
  fo.bn = bn;
  fo.n_rot = comm->rank * (sp_rows / bn);
  return gemm_wdec_launch(wfmt, W, scales, X, out_bf16, nullptr, nullptr, T, N, K, 1, nullptr, status, stream, &fo);
}

// out [T, N / 2] = silu(gate) * up for a bf16 W [N, K] whose rows are interleaved in 128-row tiles [gate | up] (the
// layout b200_unpack_fp8_bf16_gate_up writes): the activation of the feed-forward block happens in the epilogue of its
// first GEMM (pair kernel only).  comm != nullptr: X is the gathered buffer of the sequence-parallel path and the
// producer waits for the row flags (as b200_gemm_wdec_ag).
extern "C" int b200_gemm_bf16_swiglu(const void* W, const void* X, void* out_bf16, int T, int N, int K, const B200Comm* comm,
                                     int flag_rows, unsigned long long budget_ns, int* status, cudaStream_t stream) {
  if (!b200_gemm_2cta_supported(T, N, K) || !out_bf16) return -ERR_BAD_ARG;
  if (!comm) return b200_gemm_bf16_2cta(W, X, out_bf16, T, N, K, 4, nullptr, 0, 0, 0, 0, budget_ns, status, stream);
  if (comm->world <= 1 || T % comm->world || flag_rows <= 0) return -ERR_BAD_ARG;
  const int sp_rows = T / comm->world;
  if (sp_rows % 256 || sp_rows % flag_rows || sp_rows / flag_rows > B200_FLAGS_PER_SLOT) return -ERR_BAD_ARG;
  return b200_gemm_bf16_2cta(W, X, out_bf16, T, N, K, 4, comm, sp_rows, comm->rank * (sp_rows / 256), 1, flag_rows,
                             budget_ns ? budget_ns : B200_WAIT_BUDGET_NS, status, stream);
}

extern "C" int b200_splitk_reduce(const float* part, int splits, long long n, const void* residual,
                                  void* out_bf16, cudaStream_t stream) {
  const int threads = 256;
  const long long blocks = (n + threads - 1) / threads;
  splitk_reduce_kernel<<<(unsigned)blocks, threads, 0, stream>>>(
      part, splits, (size_t)n, reinterpret_cast<const __nv_bfloat16*>(residual),
      reinterpret_cast<__nv_bfloat16*>(out_bf16));
  return (int)cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Allocation-free split-K entry point (contract in no_alloc.h).
// The scratch is a device array inside this translation unit.  In host code the
// name `g_noalloc_scratch` is only a handle; the address a kernel can use comes
// from cudaGetSymbolAddress, looked up once per device with that device current.
#include "no_alloc.h"

static __device__ __align__(256) float g_noalloc_scratch[B200_NOALLOC_MAX_FLOATS];

namespace {
constexpr int kMaxDevices = 64;
float* g_noalloc_ptr[kMaxDevices] = {nullptr};
}  // namespace

extern "C" long long b200_gemm_wdec_noalloc_max_floats(void) { return B200_NOALLOC_MAX_FLOATS; }

extern "C" int b200_gemm_wdec_splitk_noalloc(int wfmt, const void* W, const float* scales, const void* X,
                                             void* out_bf16, const void* residual, int T, int N, int K,
                                             int splits, int* status, cudaStream_t stream) {
  if (T <= 0 || N <= 0 || K <= 0 || splits < 1 || !out_bf16) return -ERR_BAD_ARG;
  // same split normalisation as b200_gemm_wdec, done here so the size check sees the real count
  const int kb_total = (K + BK - 1) / BK;
  if (splits > kb_total) splits = kb_total;
  const int per = (kb_total + splits - 1) / splits;
  splits = (kb_total + per - 1) / per;
  const long long need = (long long)splits * T * N;
  if (need > B200_NOALLOC_MAX_FLOATS) {
    fprintf(stderr,
            "[b200] gemm_wdec_splitk_noalloc: splits*T*N = %d*%d*%d = %lld floats exceeds the built-in scratch "
            "of %lld floats; use fewer splits or the workspace entry point b200_gemm_wdec\n",
            splits, T, N, need, (long long)B200_NOALLOC_MAX_FLOATS);
    return B200_ERR_SCRATCH_TOO_SMALL;
  }
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -ERR_BAD_ARG;
  if (!g_noalloc_ptr[dev]) {
    // first call on this device: resolve the array's device address (device `dev` is current)
    float* ptr = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    if (!ptr) return -ERR_BAD_ARG;
    g_noalloc_ptr[dev] = ptr;
  }
  float* scratch = g_noalloc_ptr[dev];
  if (splits == 1) {
    // nothing to reduce: the plain epilogue writes bf16 (+ residual) directly
    return b200_gemm_wdec(wfmt, W, scales, X, out_bf16, nullptr, residual, T, N, K, 1, status, stream);
  }
  int rc = b200_gemm_wdec(wfmt, W, scales, X, nullptr, scratch, nullptr, T, N, K, splits, status, stream);
  if (rc != 0) return rc;
  return b200_splitk_reduce(scratch, splits, (long long)T * N, residual, out_bf16, stream);
}
