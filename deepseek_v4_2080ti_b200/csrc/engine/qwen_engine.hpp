// Native engine for the Qwen-style hybrid model, one process per GPU: with tp_world > 1 every rank loads its shard
// (heads, feed-forward width and vocabulary rows split over the ranks, row-parallel outputs summed with NCCL, arg-max
// merged over the vocabulary shards; sharding rules as cpp_engine/include/qwen_weights.hpp:15-31) and all ranks make the
// same calls in the same order (rank 0 fans requests out, see main.cpp).
// Single-GPU engine for the Qwen-style hybrid model (Gated-DeltaNet + gated GQA layers, FP8 block-128
// weights): loads a safetensors checkpoint through WeightSource, repacks the FP8 matrices on the device into the
// GEMM's tile-major layout, owns the paged KV cache / recurrent state and drives the kernel library through its
// C interface.  It implements the slot / paged-KV / batch interface the scheduler drives, so the same object
// serves the command-line tool, the persistent stdin mode and the batch scheduler.
// (Role of cpp_engine/include/qwen_engine.hpp:28-140 and cpp_engine/cuda/qwen_engine.cu.)
#pragma once
#include "qwen_target_head.hpp"
#include <cuda_runtime.h>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../core/block_pool.hpp"
#include "../core/block_table.hpp"
#include "../core/inference_engine.hpp"
#include "../core/qwen_config.hpp"
#include "../core/sampler.hpp"
#include "../core/weight_source.hpp"
#include "../comm/tp_comm.hpp"

namespace pocket {

inline void cuda_check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

// Owning device allocation.
class DeviceBuffer {
 public:
  DeviceBuffer() = default;
  explicit DeviceBuffer(size_t bytes, bool zero = false) { reset(bytes, zero); }
  DeviceBuffer(const DeviceBuffer&) = delete;
  DeviceBuffer& operator=(const DeviceBuffer&) = delete;
  DeviceBuffer(DeviceBuffer&& o) noexcept : p_(o.p_), n_(o.n_) { o.p_ = nullptr; o.n_ = 0; }
  DeviceBuffer& operator=(DeviceBuffer&& o) noexcept {
    if (this != &o) { release(); p_ = o.p_; n_ = o.n_; o.p_ = nullptr; o.n_ = 0; }
    return *this;
  }
  ~DeviceBuffer() { release(); }
  void reset(size_t bytes, bool zero = false) {
    release();
    if (bytes == 0) return;
    cuda_check(cudaMalloc(&p_, bytes), "cudaMalloc");
    n_ = bytes;
    if (zero) cuda_check(cudaMemset(p_, 0, bytes), "cudaMemset");
  }
  void release() { if (p_) cudaFree(p_); p_ = nullptr; n_ = 0; }
  template <class T = void> T* as() const { return reinterpret_cast<T*>(p_); }
  void* get() const { return p_; }
  size_t bytes() const { return n_; }
 private:
  void* p_ = nullptr;
  size_t n_ = 0;
};

// A projection ready for the GEMM kernels.
struct PackedMatrix {
  int wfmt = 0;            // 0 = bf16 row-major [N, K]; 1 = FP8 E4M3 block-128, tile-major
  int n = 0, k = 0;
  DeviceBuffer weight;
  DeviceBuffer scales;     // fp32 [ceil(N/128), ceil(K/128)] for FP8
};

struct QwenLayer {
  bool linear = false;
  DeviceBuffer in_ln, post_ln;
  PackedMatrix proj, out, gate_up, down;
  // Gated-DeltaNet
  PackedMatrix ab;
  DeviceBuffer conv_w, a_log, dt_bias, gdn_norm;
  // gated GQA
  DeviceBuffer q_norm, k_norm;
  int cache_index = 0;     // index into the per-kind state arrays
};

struct QwenEngineOptions {
  int max_slots = 1;
  int64_t max_context = 8192 + 512;
  int block_tokens = 64;
  int prefill_chunk = 8192;
  int layers = 0;          // >0: run only the first `layers` layers (smoke runs on partial checkpoints)
  int device = 0;
  std::vector<int32_t> eos_tokens;
  HostSamplingParams sampling;   // temperature 0 = greedy (arg-max on the device, 4 bytes read back per sequence)
  uint64_t seed = 0;
  // Prefix cache: > 0 keeps, at every multiple of this many tokens of a prompt (a multiple of block_tokens), the
  // sequence's KV blocks (shared by reference) and a copy of its recurrent state; a later prompt that starts with
  // the same tokens resumes from the longest such point.  Reference: the snapshot ring of the Qwen engine
  // (cpp_engine/engine/qwen_engine.cpp:5369-5563).
  int prefix_cache_interval = 0;
  int prefix_cache_entries = 4;
  int tp_world = 1, tp_rank = 0;   // tensor parallelism: this process is rank tp_rank of tp_world
  std::string nccl_id_path;        // file through which rank 0 hands the NCCL id to the others
};

struct QwenEngineStats {
  uint64_t prefix_hits = 0, prefix_tokens_reused = 0, prefix_snapshots = 0, prefix_evictions = 0;
  uint64_t kernel_launches = 0;
  double load_seconds = 0;
  size_t weight_bytes = 0, state_bytes = 0;
};

class QwenNativeEngine : public InferenceEngine {
 public:
  QwenNativeEngine(const QwenConfig& cfg, WeightSource& weights, const QwenEngineOptions& opt);
  ~QwenNativeEngine() override;

  // InferenceEngine
  int max_slots() const override { return opt_.max_slots; }
  int block_tokens() const override { return opt_.block_tokens; }
  int total_blocks() const override { return pool_->total_blocks(); }
  int64_t max_context() const override { return opt_.max_context; }
  // View of this rank's output head for drafters and other external scorers (valid while the engine lives).
  QwenTargetHead target_head() const;
  cudaStream_t stream() const { return stream_; }
  int allocate_slot() override;
  void free_slot(int slot) override;
  bool reserve(int slot, int64_t tokens) override;
  StepResult batch_prefill(const std::vector<PrefillItem>& items) override;
  StepResult batch_decode(const std::vector<int>& slots, const std::vector<int32_t>& tokens) override;
  bool is_eos(int32_t token) const override;
  int64_t vocab_size() const override { return int64_t(cfg_.vocab_size); }

  // Convenience: greedy generation for one prompt on a fresh slot.
  std::vector<int32_t> generate(const std::vector<int32_t>& prompt, int max_new_tokens, double* prefill_s = nullptr,
                                double* decode_s = nullptr);
  // Top-k (token, logit) pairs of the last forward's final row (debug / parity checks).
  std::vector<std::pair<int32_t, float>> last_topk(int k);
  int64_t slot_length(int slot) const { return lengths_.at(slot); }
  const QwenEngineStats& stats() const { return stats_; }
  const QwenConfig& config() const { return cfg_; }

 private:
  struct Scratch;
  void load(WeightSource& ws);
  // a [rows, cols] window of a checkpoint matrix (counts in elements; n < 0 = to the end)
  struct Piece { std::string name; long long row0 = 0, rows = -1, col0 = 0, cols = -1; };
  PackedMatrix load_fp8(WeightSource& ws, const std::vector<Piece>& pieces);
  PackedMatrix load_bf16(WeightSource& ws, const std::vector<Piece>& pieces);
  DeviceBuffer load_vector(WeightSource& ws, const std::string& name, bool to_f32, long long first = 0, long long count = -1);
  DeviceBuffer upload_window(const TensorView& v, size_t elem, long long row0, long long rows, long long col0, long long cols);
  void reduce_rows(void* buf, int T);
  void linear(const void* x, const PackedMatrix& w, void* out, int T, float* out_f32 = nullptr);
  void linear_stream(const void* xq, const float* inv_c, const PackedMatrix& w, void* out, int T);
  int32_t forward_prefill(int slot, const int32_t* tokens, int T, int64_t pos0, bool want_token);
  void forward_decode(const std::vector<int>& slots, const std::vector<int32_t>& tokens, std::vector<int32_t>& next);
  void upload_block_rows();
  void check_status(const char* where);
  void rc(int code, const char* what, int launches = 1);
  void sample_rows(int rows, int32_t* tokens);
  std::mt19937_64 rng_;
  std::vector<float> host_logits_;

  QwenConfig cfg_;
  QwenEngineOptions opt_;
  QwenEngineStats stats_;
  cudaStream_t stream_ = nullptr;
  int n_layers_ = 0, n_full_ = 0, n_lin_ = 0;
  int hq_ = 0, hkv_ = 0, hv_ = 0, hk_ = 0, kd_ = 0, vd_ = 0, cw_ = 0, rot_ = 0;   // per-rank head counts / widths
  int inter_ = 0, vocab_lo_ = 0, vocab_n_ = 0;                                      // per-rank feed-forward width, vocabulary rows
  TpComm tp_;
  bool stream_ok_ = false;

  std::vector<QwenLayer> layers_;
  DeviceBuffer embed_, final_norm_, inv_freq_;
  PackedMatrix lm_head_;

  std::unique_ptr<BlockPool> pool_;
  std::unique_ptr<BlockTable> table_;
  std::vector<int64_t> lengths_;
  std::vector<uint8_t> slot_used_;
  int num_blocks_ = 0, max_blocks_per_seq_ = 0;
  DeviceBuffer k_cache_, v_cache_, states_, tails_, block_table_dev_;
  size_t kv_layer_stride_ = 0, state_slot_stride_ = 0, state_layer_stride_ = 0, tail_slot_stride_ = 0,
         tail_layer_stride_ = 0;
  std::unique_ptr<Scratch> s_;

  // prefix cache
  struct PrefixEntry {
    std::vector<int32_t> tokens;       // the prefix itself (compared token by token: no hash collisions to reason about)
    std::vector<int32_t> blocks;       // tokens.size() / block_tokens KV blocks, one reference held for each
    DeviceBuffer states, tails;        // recurrent state and convolution tails after the prefix
    uint64_t stamp = 0;
  };
  std::vector<std::unique_ptr<PrefixEntry>> prefix_;
  uint64_t prefix_clock_ = 0;
  int64_t prefix_lookup(int slot, const std::vector<int32_t>& tokens);     // adopts the longest match; returns its length
  void prefix_store(int slot, const int32_t* tokens, int64_t n);
  void prefix_drop(size_t i);
 public:
  int prefix_entries() const { return int(prefix_.size()); }
};

}  // namespace pocket
