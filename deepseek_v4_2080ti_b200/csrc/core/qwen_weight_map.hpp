// Tensor-name -> (shard rule, storage kind, shape) map of the Qwen-style hybrid checkpoint, and the coverage audit
// built on it: every expected tensor present with the right dtype and shape, nothing unexpected, every sharded
// dimension divisible by the tensor-parallel world (FP8 matrices on whole 128-blocks).
// (Role of cpp_engine/include/qwen_weights.hpp:15-256, core/qwen_weight_map.cpp, tools/qwen_audit.cpp.)
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "qwen_config.hpp"
#include "safetensors_reader.hpp"

namespace pocket {

enum class QwenShardRule { Replicated, ColumnParallel, RowParallel, VocabParallel, HeadParallel };
enum class QwenLinearKind { Fp8Block128, Bf16Dense, Vector };

struct QwenTensorSpec {
  std::string name;
  std::vector<uint64_t> shape;
  std::string dtype;            // expected safetensors dtype ("F8_E4M3", "BF16"; "BF16|F32" accepts either)
  QwenShardRule rule = QwenShardRule::Replicated;
  QwenLinearKind kind = QwenLinearKind::Vector;
  int group = 1;                // rows that must stay together when the output dimension is sharded (head width)
};

const char* to_string(QwenShardRule r);

// Every tensor the runtime reads, in load order (FP8 matrices are followed by their ".weight_scale_inv").
std::vector<QwenTensorSpec> qwen_expected_tensors(const QwenConfig& cfg);
std::vector<QwenTensorSpec> qwen_mtp_tensors(const QwenConfig& cfg);

// Shape of rank `rank`'s slice of a tensor under tensor parallelism of size `world`.
std::vector<uint64_t> qwen_shard_shape(const QwenTensorSpec& spec, int world, int rank);

struct QwenAuditReport {
  size_t expected = 0, found = 0;
  bool has_mtp = false;     // the checkpoint carries mtp.* tensors, so the whole MTP head was required
  uint64_t bytes = 0;
  std::vector<std::string> missing, unexpected, wrong_shape, wrong_dtype, not_divisible;
  bool ok(bool strict) const {
    return missing.empty() && wrong_shape.empty() && wrong_dtype.empty() && not_divisible.empty() && (!strict || unexpected.empty());
  }
};

QwenAuditReport qwen_audit(SafetensorsModel& model, const QwenConfig& cfg, int tp_world = 1);

}  // namespace pocket
