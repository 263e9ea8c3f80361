#include "model_config.hpp"

#include <sstream>
#include <stdexcept>

#include "qwen_config.hpp"   // read_text_file

namespace pocket {
namespace {

using C = MoeModelConfig;
enum class Kind { U64, F64 };

struct Field {
  const char* name;                  // printed name
  Kind kind;
  uint64_t C::*u;
  double C::*f;
  const char* gguf;                  // key suffix under the architecture prefix ("" = none)
  const char* json[3];               // accepted config.json spellings, first match wins
};

constexpr Field U(const char* n, uint64_t C::*m, const char* g, const char* j0, const char* j1 = nullptr,
                  const char* j2 = nullptr) { return Field{n, Kind::U64, m, nullptr, g, {j0, j1, j2}}; }
constexpr Field F(const char* n, double C::*m, const char* g, const char* j0, const char* j1 = nullptr,
                  const char* j2 = nullptr) { return Field{n, Kind::F64, nullptr, m, g, {j0, j1, j2}}; }

const Field kFields[] = {
    U("vocab_size", &C::vocab_size, "vocab_size", "vocab_size"),
    U("dim", &C::dim, "embedding_length", "hidden_size", "dim"),
    U("n_layers", &C::n_layers, "block_count", "num_hidden_layers", "n_layers"),
    U("n_dense_layers", &C::n_dense_layers, "leading_dense_block_count", "first_k_dense_replace", "n_dense_layers"),
    U("n_heads", &C::n_heads, "attention.head_count", "num_attention_heads", "n_heads"),
    U("kv_heads", &C::kv_heads, "attention.head_count_kv", "num_key_value_heads"),
    U("head_dim", &C::head_dim, "attention.key_length", "head_dim", "qk_head_dim"),
    U("value_dim", &C::value_dim, "attention.value_length", "v_head_dim"),
    U("q_lora_rank", &C::q_lora_rank, "attention.q_lora_rank", "q_lora_rank"),
    U("kv_lora_rank", &C::kv_lora_rank, "attention.kv_lora_rank", "kv_lora_rank"),
    U("o_lora_rank", &C::o_lora_rank, "attention.output_lora_rank", "o_lora_rank"),
    U("o_groups", &C::o_groups, "attention.output_group_count", "o_groups"),
    U("index_n_heads", &C::index_n_heads, "attention.indexer.head_count", "index_n_heads"),
    U("index_head_dim", &C::index_head_dim, "attention.indexer.key_length", "index_head_dim"),
    U("index_topk", &C::index_topk, "attention.indexer.top_k", "index_topk"),
    U("n_routed_experts", &C::n_routed_experts, "expert_count", "n_routed_experts", "num_local_experts", "num_experts"),
    U("n_shared_experts", &C::n_shared_experts, "expert_shared_count", "n_shared_experts"),
    U("n_activated_experts", &C::n_activated_experts, "expert_used_count", "num_experts_per_tok", "n_activated_experts"),
    U("moe_inter_dim", &C::moe_inter_dim, "expert_feed_forward_length", "moe_intermediate_size", "moe_inter_dim"),
    U("inter_dim", &C::inter_dim, "feed_forward_length", "intermediate_size", "inter_dim"),
    F("route_scale", &C::route_scale, "expert_weights_scale", "routed_scaling_factor", "route_scale"),
    F("swiglu_limit", &C::swiglu_limit, "swiglu_limit", "swiglu_limit"),
    F("rms_norm_eps", &C::rms_norm_eps, "attention.layer_norm_rms_epsilon", "rms_norm_eps"),
    U("context_length", &C::context_length, "context_length", "max_position_embeddings", "max_seq_len"),
    U("original_context_length", &C::original_context_length, "rope.scaling.original_context_length",
      "original_max_position_embeddings", "original_seq_len"),
    U("rope_dim", &C::rope_dim, "rope.dimension_count", "qk_rope_head_dim", "rope_head_dim"),
    F("rope_theta", &C::rope_theta, "rope.freq_base", "rope_theta"),
    F("rope_factor", &C::rope_factor, "rope.scaling.factor", "rope_factor"),
    F("beta_fast", &C::beta_fast, "rope.scaling.yarn_beta_fast", "beta_fast"),
    F("beta_slow", &C::beta_slow, "rope.scaling.yarn_beta_slow", "beta_slow"),
    U("window_size", &C::window_size, "attention.sliding_window", "sliding_window", "window_size"),
    F("compress_rope_theta", &C::compress_rope_theta, "attention.compress_rope_freq_base", "compress_rope_theta"),
    U("n_hash_layers", &C::n_hash_layers, "hash_layer_count", "num_hash_layers", "n_hash_layers"),
    U("hc_mult", &C::hc_mult, "hyper_connection.count", "hc_mult"),
    U("hc_sinkhorn_iters", &C::hc_sinkhorn_iters, "hyper_connection.sinkhorn_iterations", "hc_sinkhorn_iters"),
    U("n_mtp_layers", &C::n_mtp_layers, "nextn_predict_layers", "num_nextn_predict_layers", "n_mtp_layers"),
};

const char* const kFallbackPrefixes[] = {"deepseek4.", "llama."};

const GGUFValue* lookup(const GGUFReader& g, const std::string& arch, const char* suffix) {
  if (!*suffix) return nullptr;
  if (!arch.empty())
    if (const GGUFValue* v = g.find(arch + "." + suffix)) return v;
  for (const char* p : kFallbackPrefixes)
    if (const GGUFValue* v = g.find(std::string(p) + suffix)) return v;
  return nullptr;
}

bool scalar(const GGUFValue& v) {
  using K = GGUFValue::Kind;
  return v.kind == K::UInt || v.kind == K::Int || v.kind == K::Float || v.kind == K::Bool;
}

template <class T>
std::string join(const std::vector<T>& v) {
  std::ostringstream o;
  for (size_t i = 0; i < v.size(); ++i) o << (i ? "," : "") << v[i];
  return o.str();
}

}  // namespace

MoeModelConfig MoeModelConfig::from_gguf(const GGUFReader& g) {
  MoeModelConfig c;
  c.architecture = g.get_string("general.architecture");
  for (const Field& f : kFields) {
    const GGUFValue* v = lookup(g, c.architecture, f.gguf);
    if (!v || !scalar(*v)) continue;
    if (f.kind == Kind::U64) c.*(f.u) = static_cast<uint64_t>(v->as_int());
    else c.*(f.f) = v->as_float();
  }
  if (c.vocab_size == 0)
    if (const GGUFValue* toks = g.find("tokenizer.ggml.tokens"))
      if (toks->kind == GGUFValue::Kind::Array) c.vocab_size = toks->items.size();
  if (const GGUFValue* r = lookup(g, c.architecture, "attention.compress_ratios"))
    if (r->kind == GGUFValue::Kind::Array)
      for (const auto& it : r->items) c.compress_ratios.push_back(static_cast<uint64_t>(it.as_int()));
  if (const GGUFValue* r = lookup(g, c.architecture, "swiglu_clamp_exp"))
    if (r->kind == GGUFValue::Kind::Array)
      for (const auto& it : r->items) c.swiglu_clamp_exp.push_back(it.as_float());
  return c;
}

MoeModelConfig MoeModelConfig::from_hf_json(const Json& root) {
  if (!root.is_object()) throw std::runtime_error("model config: the document is not a JSON object");
  // multimodal wrappers keep the language model under text_config
  const Json& t = root["text_config"].is_object() ? root["text_config"] : root;
  MoeModelConfig c;
  c.architecture = t["model_type"].is_string() ? t["model_type"].as_string() : root["model_type"].as_string();
  const Json& scaling = t["rope_scaling"];
  for (const Field& f : kFields) {
    const Json* v = nullptr;
    for (const char* k : f.json) {
      if (!k) break;
      if ((v = t.find(k)) && v->is_number()) break;
      if (scaling.is_object() && (v = scaling.find(k)) && v->is_number()) break;
      v = nullptr;
    }
    if (!v) continue;
    if (f.kind == Kind::U64) c.*(f.u) = static_cast<uint64_t>(v->as_int());
    else c.*(f.f) = v->as_double();
  }
  if (scaling.is_object() && c.rope_factor == 0.0) c.rope_factor = scaling["factor"].as_double(0.0);
  for (const Json& r : t["compress_ratios"].items()) c.compress_ratios.push_back(static_cast<uint64_t>(r.as_int()));
  for (const Json& r : t["swiglu_clamp_exp"].items()) c.swiglu_clamp_exp.push_back(r.as_double());
  return c;
}

MoeModelConfig MoeModelConfig::from_hf_dir(const std::string& dir) {
  return from_hf_json(Json::parse(read_text_file(dir + "/config.json")));
}

std::string MoeModelConfig::describe() const {
  std::ostringstream o;
  o << "architecture=" << (architecture.empty() ? "?" : architecture);
  for (const Field& f : kFields) {
    if (f.kind == Kind::U64) { if (this->*(f.u)) o << " " << f.name << "=" << this->*(f.u); }
    else if (this->*(f.f) != 0.0) o << " " << f.name << "=" << this->*(f.f);
  }
  if (!compress_ratios.empty()) o << " compress_ratios=" << join(compress_ratios);
  if (!swiglu_clamp_exp.empty()) o << " swiglu_clamp_exp=" << join(swiglu_clamp_exp);
  return o.str();
}

Json MoeModelConfig::to_json() const {
  Json j = Json::object();
  j.set("architecture", architecture);
  for (const Field& f : kFields) {
    if (f.kind == Kind::U64) j.set(f.name, static_cast<int64_t>(this->*(f.u)));
    else j.set(f.name, this->*(f.f));
  }
  Json r = Json::array();
  for (uint64_t v : compress_ratios) r.push_back(static_cast<int64_t>(v));
  j.set("compress_ratios", r);
  Json e = Json::array();
  for (double v : swiglu_clamp_exp) e.push_back(v);
  j.set("swiglu_clamp_exp", e);
  return j;
}

std::vector<std::string> MoeModelConfig::problems(int tp, int ep) const {
  std::vector<std::string> p;
  auto need = [&](bool ok, const std::string& what) { if (!ok) p.push_back(what); };
  need(dim > 0, "dim is missing");
  need(n_layers > 0, "n_layers is missing");
  need(n_heads > 0, "n_heads is missing");
  need(vocab_size > 0, "vocab_size is missing (no field and no tokenizer.ggml.tokens)");
  if (tp > 1) {
    need(n_heads % tp == 0, "n_heads " + std::to_string(n_heads) + " does not divide over " + std::to_string(tp) + " ranks");
    if (!is_mla() && kv_heads)
      need(kv_heads % tp == 0 || tp % kv_heads == 0, "kv_heads " + std::to_string(kv_heads) + " neither divides nor is divided by " + std::to_string(tp));
    if (index_n_heads) need(index_n_heads % tp == 0 || tp % index_n_heads == 0, "index_n_heads does not split over the ranks");
    if (o_groups) need(o_groups % tp == 0, "o_groups " + std::to_string(o_groups) + " does not divide over " + std::to_string(tp) + " ranks");
  }
  if (n_routed_experts) {
    need(n_activated_experts > 0 && n_activated_experts <= n_routed_experts, "n_activated_experts must be in 1..n_routed_experts");
    need(moe_inter_dim > 0, "moe_inter_dim is missing");
    if (ep > 1) need(n_routed_experts % ep == 0, "n_routed_experts " + std::to_string(n_routed_experts) + " does not divide over " + std::to_string(ep) + " expert ranks");
  }
  if (has_indexer()) need(index_head_dim > 0, "index_head_dim is missing");
  if (!compress_ratios.empty())
    need(compress_ratios.size() == n_layers, "compress_ratios has " + std::to_string(compress_ratios.size()) + " entries for " + std::to_string(n_layers) + " layers");
  if (rope_factor > 1.0) need(original_context_length > 0, "rope scaling without original_context_length");
  return p;
}

uint64_t MoeModelConfig::kv_bytes_per_token_layer() const {
  if (kv_lora_rank) return 2 * (kv_lora_rank + rope_dim);
  const uint64_t heads = kv_heads ? kv_heads : n_heads;
  return 2 * heads * (head_dim + (value_dim ? value_dim : head_dim));
}

}  // namespace pocket
