// Non-owning view of the target model's vocabulary-parallel output head, for code outside the engine that has to
// score hidden states with the target's own lm_head (external drafters, verification of a draft's hidden state)
// without knowing how the checkpoint stores it: bf16 row-major or FP8 block-128, full or a vocabulary shard.
// Reference: cpp_engine/include/qwen_target_head.hpp (QwenTargetHeadAdapter: kind, weight, scale, local_vocab,
// hidden_size, vocab_start, project_f16_to_f32).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "../kernels/ops.h"

namespace pocket {

struct QwenTargetHead {
  int wfmt = 0;                  // 0 = bf16 [local_vocab, hidden]; 1 = FP8 E4M3 block-128, tile-major
  const void* weight = nullptr;
  const float* scales = nullptr; // fp32 [ceil(local_vocab / 128), ceil(hidden / 128)] for FP8
  int local_vocab = 0, hidden = 0;
  int64_t vocab_start = 0;       // first vocabulary id of this rank's shard
  int* status = nullptr;         // the engine's device error word

  bool valid() const {
    return weight && local_vocab > 0 && hidden > 0 && hidden % 16 == 0 && status && (wfmt == 0 || (wfmt == 1 && scales));
  }
  // hidden_bf16 [rows, hidden] -> logits fp32 [rows, local_vocab] on `stream`.  Returns 0 or the kernel library's code.
  int project(const void* hidden_bf16, float* logits, int rows, cudaStream_t stream) const {
    if (!valid() || !hidden_bf16 || !logits || rows <= 0) return -6;
    return b200_gemm_wdec_ex(wfmt, weight, scales, hidden_bf16, nullptr, logits, nullptr, rows, local_vocab, hidden, 1,
                             nullptr, status, stream);
  }
  // Global vocabulary id of a column of this shard's logits.
  int64_t token_of(int column) const { return vocab_start + column; }
};

}  // namespace pocket
