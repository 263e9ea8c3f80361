// Model configuration structs parsed from JSON: the Qwen-style hybrid text config
// (Qwen3_5ForConditionalGeneration, cpp_engine/core/qwen_config.cpp:150-240) and the
// DeepSeek-style config (configs/config.json:1-34, cpp_engine/core/model_config.cpp).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "json_lite.hpp"

namespace pocket {

struct QwenConfig {
  int64_t vocab_size = 0, hidden_size = 0, intermediate_size = 0, num_hidden_layers = 0;
  int64_t num_attention_heads = 0, num_key_value_heads = 0, head_dim = 0;
  bool attn_output_gate = true;
  int64_t linear_num_key_heads = 0, linear_num_value_heads = 0, linear_key_head_dim = 0, linear_value_head_dim = 0;
  int64_t linear_conv_kernel_dim = 4, max_position_embeddings = 0;
  double rms_norm_eps = 1e-6, partial_rotary_factor = 1.0, rope_theta = 10000.0;
  std::vector<std::string> layer_types;
  std::string quant_method;          // "fp8" when quantization_config says so
  int64_t quant_block = 0;           // weight_block_size[0]
  int64_t num_full_layers() const;
  int64_t num_linear_layers() const;
  int64_t rotary_dim() const { return static_cast<int64_t>(head_dim * partial_rotary_factor); }
  // Throws std::runtime_error listing every problem (missing fields, head/TP divisibility).
  void validate(int tp_world = 1) const;
  static QwenConfig from_json(const Json& root);
  static QwenConfig from_file(const std::string& path);
  static bool is_qwen3_5(const Json& root);
};

struct DeepSeekConfig {
  int64_t vocab_size = 0, dim = 0, n_layers = 0, n_dense_layers = 0, n_heads = 0, inter_dim = 0, moe_inter_dim = 0;
  int64_t n_routed_experts = 0, n_shared_experts = 0, n_activated_experts = 0;
  int64_t q_lora_rank = 0, kv_lora_rank = 0, qk_nope_head_dim = 0, qk_rope_head_dim = 0, v_head_dim = 0;
  int64_t index_n_heads = 0, index_head_dim = 0, index_topk = 0;
  double route_scale = 1.0, rope_theta = 10000.0, rope_factor = 1.0, rms_norm_eps = 1e-6;
  std::string score_func = "softmax", dtype = "bf16", expert_dtype = "fp4", scale_fmt = "ue8m0";
  int64_t n_mtp_layers = 0;
  static DeepSeekConfig from_json(const Json& root);
  static DeepSeekConfig from_file(const std::string& path);
};

std::string read_text_file(const std::string& path);

}  // namespace pocket
