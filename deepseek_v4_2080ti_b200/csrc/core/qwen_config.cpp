#include "qwen_config.hpp"

#include <fstream>
#include <sstream>
#include <stdexcept>

namespace pocket {

std::string read_text_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) throw std::runtime_error("cannot read " + path);
  std::stringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

bool QwenConfig::is_qwen3_5(const Json& root) {
  for (const auto& a : root["architectures"].items())
    if (a.as_string().rfind("Qwen3_5", 0) == 0) return true;
  const std::string mt = root["model_type"].as_string();
  return mt == "qwen3_5" || mt == "qwen3_5_text";
}

QwenConfig QwenConfig::from_json(const Json& root) {
  const Json& t = root.contains("text_config") ? root["text_config"] : root;
  QwenConfig c;
  auto I = [&](const char* k, int64_t d = 0) { return t[k].as_int(d); };
  c.vocab_size = I("vocab_size");
  c.hidden_size = I("hidden_size");
  c.intermediate_size = I("intermediate_size");
  c.num_hidden_layers = I("num_hidden_layers");
  c.num_attention_heads = I("num_attention_heads");
  c.num_key_value_heads = I("num_key_value_heads", c.num_attention_heads);
  c.head_dim = I("head_dim", c.num_attention_heads ? c.hidden_size / c.num_attention_heads : 0);
  c.attn_output_gate = t["attn_output_gate"].as_bool(true);
  c.linear_num_key_heads = I("linear_num_key_heads");
  c.linear_num_value_heads = I("linear_num_value_heads");
  c.linear_key_head_dim = I("linear_key_head_dim");
  c.linear_value_head_dim = I("linear_value_head_dim");
  c.linear_conv_kernel_dim = I("linear_conv_kernel_dim", 4);
  c.max_position_embeddings = I("max_position_embeddings");
  c.rms_norm_eps = t["rms_norm_eps"].as_double(1e-6);
  c.partial_rotary_factor = t["partial_rotary_factor"].as_double(1.0);
  c.rope_theta = t["rope_theta"].as_double(10000.0);
  const Json& rp = t["rope_parameters"];
  if (rp.is_object()) {
    if (rp.contains("rope_theta")) c.rope_theta = rp["rope_theta"].as_double(c.rope_theta);
    if (rp.contains("partial_rotary_factor")) c.partial_rotary_factor = rp["partial_rotary_factor"].as_double(c.partial_rotary_factor);
  }
  for (const auto& l : t["layer_types"].items()) c.layer_types.push_back(l.as_string());
  if (c.layer_types.empty()) {
    const int64_t every = I("full_attention_interval", 4);
    for (int64_t i = 0; i < c.num_hidden_layers; ++i)
      c.layer_types.push_back(((i + 1) % every == 0) ? "full_attention" : "linear_attention");
  }
  const Json& q = root.contains("quantization_config") ? root["quantization_config"] : t["quantization_config"];
  if (q.is_object()) {
    c.quant_method = q["quant_method"].as_string();
    c.quant_block = q["weight_block_size"][0].as_int(0);
  }
  return c;
}

QwenConfig QwenConfig::from_file(const std::string& path) { return from_json(Json::parse(read_text_file(path))); }

int64_t QwenConfig::num_full_layers() const {
  int64_t n = 0;
  for (const auto& l : layer_types) n += l == "full_attention";
  return n;
}
int64_t QwenConfig::num_linear_layers() const { return static_cast<int64_t>(layer_types.size()) - num_full_layers(); }

void QwenConfig::validate(int tp) const {
  std::string err;
  auto need = [&](bool ok, const std::string& m) { if (!ok) err += (err.empty() ? "" : "; ") + m; };
  need(vocab_size > 0, "vocab_size missing");
  need(hidden_size > 0, "hidden_size missing");
  need(num_hidden_layers > 0, "num_hidden_layers missing");
  need(static_cast<int64_t>(layer_types.size()) == num_hidden_layers, "layer_types length != num_hidden_layers");
  need(num_attention_heads > 0 && num_key_value_heads > 0, "attention heads missing");
  need(num_key_value_heads == 0 || num_attention_heads % num_key_value_heads == 0, "q heads not a multiple of kv heads");
  if (num_linear_layers() > 0) {
    need(linear_num_key_heads > 0 && linear_num_value_heads > 0, "linear attention heads missing");
    need(linear_num_key_heads == 0 || linear_num_value_heads % linear_num_key_heads == 0, "linear value heads not a multiple of key heads");
  }
  for (const auto& l : layer_types) need(l == "full_attention" || l == "linear_attention", "unknown layer type " + l);
  if (tp > 1) {
    need(num_attention_heads % tp == 0, "num_attention_heads not divisible by tp");
    need(num_key_value_heads % tp == 0, "num_key_value_heads not divisible by tp");
    need(linear_num_key_heads % tp == 0, "linear_num_key_heads not divisible by tp");
    need(linear_num_value_heads % tp == 0, "linear_num_value_heads not divisible by tp");
    need(intermediate_size % (128 * tp) == 0, "intermediate_size / tp must keep whole 128-wide scale blocks");
  }
  if (!err.empty()) throw std::runtime_error("qwen config: " + err);
}

DeepSeekConfig DeepSeekConfig::from_json(const Json& t) {
  DeepSeekConfig c;
  auto I = [&](const char* k, int64_t d = 0) { return t[k].as_int(d); };
  c.vocab_size = I("vocab_size");
  c.dim = I("dim");
  c.n_layers = I("n_layers");
  c.n_dense_layers = I("n_dense_layers");
  c.n_heads = I("n_heads");
  c.inter_dim = I("inter_dim");
  c.moe_inter_dim = I("moe_inter_dim");
  c.n_routed_experts = I("n_routed_experts");
  c.n_shared_experts = I("n_shared_experts");
  c.n_activated_experts = I("n_activated_experts");
  c.q_lora_rank = I("q_lora_rank");
  c.kv_lora_rank = I("kv_lora_rank");
  c.qk_nope_head_dim = I("qk_nope_head_dim");
  c.qk_rope_head_dim = I("qk_rope_head_dim");
  c.v_head_dim = I("v_head_dim");
  c.index_n_heads = I("index_n_heads");
  c.index_head_dim = I("index_head_dim");
  c.index_topk = I("index_topk");
  c.route_scale = t["route_scale"].as_double(1.0);
  c.rope_theta = t["rope_theta"].as_double(10000.0);
  c.rope_factor = t["rope_factor"].as_double(1.0);
  c.rms_norm_eps = t["rms_norm_eps"].as_double(1e-6);
  if (t["score_func"].is_string()) c.score_func = t["score_func"].as_string();
  if (t["dtype"].is_string()) c.dtype = t["dtype"].as_string();
  if (t["expert_dtype"].is_string()) c.expert_dtype = t["expert_dtype"].as_string();
  if (t["scale_fmt"].is_string()) c.scale_fmt = t["scale_fmt"].as_string();
  c.n_mtp_layers = I("n_mtp_layers");
  return c;
}

DeepSeekConfig DeepSeekConfig::from_file(const std::string& path) { return from_json(Json::parse(read_text_file(path))); }

}  // namespace pocket
