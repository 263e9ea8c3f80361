// Architecture-neutral description of a sparse-attention MoE checkpoint (DeepSeek-V4, GLM-DSA, MiniMax-M2 ...),
// filled either from the metadata of a GGUF file or from a Hugging Face style config.json.  One table names every
// field once (struct member, GGUF key suffix, JSON keys), so the two readers, the printer and the checks cannot
// drift apart.  Same role as the reference's cpp_engine/core/model_config.cpp (ModelConfig::from_gguf,
// ModelConfig::from_hf_config, ModelConfig::to_string).
#pragma once
#include <cstdint>
#include <string>
#include <vector>

#include "gguf_reader.hpp"
#include "json_lite.hpp"

namespace pocket {

struct MoeModelConfig {
  std::string architecture;                 // general.architecture / model_type
  uint64_t vocab_size = 0, dim = 0, n_layers = 0, n_heads = 0, kv_heads = 0, head_dim = 0, value_dim = 0;
  uint64_t q_lora_rank = 0, kv_lora_rank = 0, o_lora_rank = 0, o_groups = 0;
  uint64_t index_n_heads = 0, index_head_dim = 0, index_topk = 0;
  uint64_t n_routed_experts = 0, n_shared_experts = 0, n_activated_experts = 0, moe_inter_dim = 0, inter_dim = 0;
  uint64_t n_dense_layers = 0;
  double route_scale = 0.0, swiglu_limit = 0.0, rms_norm_eps = 0.0;
  uint64_t context_length = 0, original_context_length = 0, rope_dim = 0;
  double rope_theta = 0.0, rope_factor = 0.0, beta_fast = 0.0, beta_slow = 0.0;
  uint64_t window_size = 0;
  double compress_rope_theta = 0.0;
  uint64_t n_hash_layers = 0, hc_mult = 0, hc_sinkhorn_iters = 0, n_mtp_layers = 0;
  std::vector<uint64_t> compress_ratios;    // per layer: 0 / 1 = uncompressed
  std::vector<double> swiglu_clamp_exp;

  // Metadata keys are looked up as "<general.architecture>.<suffix>", then under the fallback prefixes
  // "deepseek4." and "llama." (files converted by older tools).  The vocabulary size falls back to the length of
  // tokenizer.ggml.tokens.
  static MoeModelConfig from_gguf(const GGUFReader& file);
  // config.json of the checkpoint; rope_scaling{factor, beta_fast, beta_slow, original_max_position_embeddings}
  // is read when present.  Both the Hugging Face spellings and the short spellings of the DeepSeek inference
  // config (dim, n_layers, n_heads ...) are accepted.
  static MoeModelConfig from_hf_json(const Json& root);
  static MoeModelConfig from_hf_dir(const std::string& ckpt_dir);   // <dir>/config.json
  // One "name=value" pair per field that is set, in table order; lists as a,b,c.
  std::string describe() const;
  Json to_json() const;
  // Problems that make the shape unusable on tp_world x ep_world ranks (empty = fine).
  std::vector<std::string> problems(int tp_world = 1, int ep_world = 1) const;
  bool has_indexer() const { return index_n_heads > 0 && index_topk > 0; }
  bool is_mla() const { return kv_lora_rank > 0 || q_lora_rank > 0; }
  // Latent-cache bytes per token and layer at 2-byte elements: kv_lora_rank + rope_dim for MLA, else
  // kv_heads x (head_dim + value_dim).
  uint64_t kv_bytes_per_token_layer() const;
};

}  // namespace pocket
