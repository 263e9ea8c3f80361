#include "qwen_weight_map.hpp"

#include <algorithm>
#include <set>

namespace pocket {

const char* to_string(QwenShardRule r) {
  switch (r) {
    case QwenShardRule::Replicated: return "replicated";
    case QwenShardRule::ColumnParallel: return "column_parallel";
    case QwenShardRule::RowParallel: return "row_parallel";
    case QwenShardRule::VocabParallel: return "vocab_parallel";
    case QwenShardRule::HeadParallel: return "head_parallel";
  }
  return "?";
}

namespace {

void fp8(std::vector<QwenTensorSpec>& out, const std::string& base, uint64_t n, uint64_t k, QwenShardRule rule, int group) {
  out.push_back({base + ".weight", {n, k}, "F8_E4M3", rule, QwenLinearKind::Fp8Block128, group});
  out.push_back({base + ".weight_scale_inv", {(n + 127) / 128, (k + 127) / 128}, "BF16|F32", rule, QwenLinearKind::Fp8Block128,
                 std::max(1, group / 128)});
}

}  // namespace

std::vector<QwenTensorSpec> qwen_expected_tensors(const QwenConfig& c) {
  std::vector<QwenTensorSpec> out;
  const uint64_t h = uint64_t(c.hidden_size), inter = uint64_t(c.intermediate_size), v = uint64_t(c.vocab_size);
  const uint64_t d = uint64_t(c.head_dim);
  const uint64_t kd = uint64_t(c.linear_num_key_heads * c.linear_key_head_dim);
  const uint64_t vd = uint64_t(c.linear_num_value_heads * c.linear_value_head_dim);
  const uint64_t hv = uint64_t(c.linear_num_value_heads);
  const uint64_t qd = uint64_t(c.num_attention_heads) * d, kvd = uint64_t(c.num_key_value_heads) * d;
  const std::string root = "model.language_model.";
  out.push_back({root + "embed_tokens.weight", {v, h}, "BF16", QwenShardRule::VocabParallel, QwenLinearKind::Bf16Dense, 1});
  out.push_back({root + "norm.weight", {h}, "BF16", QwenShardRule::Replicated, QwenLinearKind::Vector, 1});
  out.push_back({"lm_head.weight", {v, h}, "BF16", QwenShardRule::VocabParallel, QwenLinearKind::Bf16Dense, 1});
  for (int64_t i = 0; i < c.num_hidden_layers; ++i) {
    const std::string p = root + "layers." + std::to_string(i) + ".";
    out.push_back({p + "input_layernorm.weight", {h}, "BF16", QwenShardRule::Replicated, QwenLinearKind::Vector, 1});
    out.push_back({p + "post_attention_layernorm.weight", {h}, "BF16", QwenShardRule::Replicated, QwenLinearKind::Vector, 1});
    if (c.layer_types.at(size_t(i)) == "linear_attention") {
      const std::string a = p + "linear_attn.";
      // q | k | v row ranges are sharded separately (each by heads), so the fused matrix is "head parallel"
      fp8(out, a + "in_proj_qkv", 2 * kd + vd, h, QwenShardRule::HeadParallel, int(c.linear_key_head_dim));
      fp8(out, a + "in_proj_z", vd, h, QwenShardRule::ColumnParallel, int(c.linear_value_head_dim));
      fp8(out, a + "out_proj", h, vd, QwenShardRule::RowParallel, int(c.linear_value_head_dim));
      out.push_back({a + "in_proj_a.weight", {hv, h}, "BF16", QwenShardRule::ColumnParallel, QwenLinearKind::Bf16Dense, 1});
      out.push_back({a + "in_proj_b.weight", {hv, h}, "BF16", QwenShardRule::ColumnParallel, QwenLinearKind::Bf16Dense, 1});
      out.push_back({a + "conv1d.weight", {2 * kd + vd, 1, uint64_t(c.linear_conv_kernel_dim)}, "BF16", QwenShardRule::HeadParallel,
                     QwenLinearKind::Vector, int(c.linear_key_head_dim)});
      out.push_back({a + "A_log", {hv}, "BF16|F32", QwenShardRule::ColumnParallel, QwenLinearKind::Vector, 1});
      out.push_back({a + "dt_bias", {hv}, "BF16|F32", QwenShardRule::ColumnParallel, QwenLinearKind::Vector, 1});
      out.push_back({a + "norm.weight", {uint64_t(c.linear_value_head_dim)}, "BF16", QwenShardRule::Replicated, QwenLinearKind::Vector, 1});
    } else {
      const std::string a = p + "self_attn.";
      fp8(out, a + "q_proj", qd * (c.attn_output_gate ? 2 : 1), h, QwenShardRule::ColumnParallel, int(d) * (c.attn_output_gate ? 2 : 1));
      fp8(out, a + "k_proj", kvd, h, QwenShardRule::ColumnParallel, int(d));
      fp8(out, a + "v_proj", kvd, h, QwenShardRule::ColumnParallel, int(d));
      fp8(out, a + "o_proj", h, qd, QwenShardRule::RowParallel, int(d));
      out.push_back({a + "q_norm.weight", {d}, "BF16", QwenShardRule::Replicated, QwenLinearKind::Vector, 1});
      out.push_back({a + "k_norm.weight", {d}, "BF16", QwenShardRule::Replicated, QwenLinearKind::Vector, 1});
    }
    fp8(out, p + "mlp.gate_proj", inter, h, QwenShardRule::ColumnParallel, 128);
    fp8(out, p + "mlp.up_proj", inter, h, QwenShardRule::ColumnParallel, 128);
    fp8(out, p + "mlp.down_proj", h, inter, QwenShardRule::RowParallel, 128);
  }
  return out;
}

// The multi-token-prediction head: embedding and hidden state are normalised separately, concatenated and fused by
// ``mtp.fc`` [H, 2H], then one full-attention decoder layer and ``mtp.norm`` feed the shared lm_head.  Its matrices
// may be FP8 block-scaled like the trunk or plain BF16.
std::vector<QwenTensorSpec> qwen_mtp_tensors(const QwenConfig& c) {
  std::vector<QwenTensorSpec> out;
  const uint64_t h = uint64_t(c.hidden_size), inter = uint64_t(c.intermediate_size), d = uint64_t(c.head_dim);
  const uint64_t qd = uint64_t(c.num_attention_heads) * d, kvd = uint64_t(c.num_key_value_heads) * d;
  auto vec = [&](const std::string& n, uint64_t len) {
    out.push_back({n, {len}, "BF16", QwenShardRule::Replicated, QwenLinearKind::Vector, 1});
  };
  auto lin = [&](const std::string& base, uint64_t n, uint64_t k, QwenShardRule rule, int group) {
    const size_t first = out.size();
    fp8(out, base, n, k, rule, group);
    out[first].dtype = "F8_E4M3|BF16";
  };
  vec("mtp.pre_fc_norm_embedding.weight", h);
  vec("mtp.pre_fc_norm_hidden.weight", h);
  vec("mtp.norm.weight", h);
  lin("mtp.fc", h, 2 * h, QwenShardRule::Replicated, 1);
  const std::string p = "mtp.layers.0.";
  vec(p + "input_layernorm.weight", h);
  vec(p + "post_attention_layernorm.weight", h);
  const int qgroup = int(d) * (c.attn_output_gate ? 2 : 1);
  lin(p + "self_attn.q_proj", qd * (c.attn_output_gate ? 2 : 1), h, QwenShardRule::ColumnParallel, qgroup);
  lin(p + "self_attn.k_proj", kvd, h, QwenShardRule::ColumnParallel, int(d));
  lin(p + "self_attn.v_proj", kvd, h, QwenShardRule::ColumnParallel, int(d));
  lin(p + "self_attn.o_proj", h, qd, QwenShardRule::RowParallel, int(d));
  vec(p + "self_attn.q_norm.weight", d);
  vec(p + "self_attn.k_norm.weight", d);
  lin(p + "mlp.gate_proj", inter, h, QwenShardRule::ColumnParallel, 128);
  lin(p + "mlp.up_proj", inter, h, QwenShardRule::ColumnParallel, 128);
  lin(p + "mlp.down_proj", h, inter, QwenShardRule::RowParallel, 128);
  return out;
}

std::vector<uint64_t> qwen_shard_shape(const QwenTensorSpec& s, int world, int rank) {
  std::vector<uint64_t> shape = s.shape;
  if (world <= 1) return shape;
  switch (s.rule) {
    case QwenShardRule::Replicated: break;
    case QwenShardRule::VocabParallel: {
      const uint64_t per = (shape[0] + uint64_t(world) - 1) / uint64_t(world);
      const uint64_t lo = std::min(shape[0], per * uint64_t(rank));
      shape[0] = std::min(shape[0], lo + per) - lo;
      break;
    }
    case QwenShardRule::ColumnParallel:
    case QwenShardRule::HeadParallel:
      shape[0] /= uint64_t(world);
      break;
    case QwenShardRule::RowParallel:
      if (shape.size() >= 2) shape[1] /= uint64_t(world);
      break;
  }
  return shape;
}

QwenAuditReport qwen_audit(SafetensorsModel& model, const QwenConfig& cfg, int tp_world) {
  QwenAuditReport rep;
  std::vector<QwenTensorSpec> specs = qwen_expected_tensors(cfg);
  for (const std::string& n : model.names())
    if (n.compare(0, 4, "mtp.") == 0) {                  // a checkpoint with an MTP head must have all of it
      const std::vector<QwenTensorSpec> mtp = qwen_mtp_tensors(cfg);
      specs.insert(specs.end(), mtp.begin(), mtp.end());
      rep.has_mtp = true;
      break;
    }
  rep.expected = specs.size();
  std::set<std::string> known;
  for (const QwenTensorSpec& s : specs) {
    known.insert(s.name);
    const uint8_t* base = nullptr;
    const SafeTensorInfo* info = model.find(s.name, &base);
    if (!info) {
      if (s.name == "lm_head.weight") continue;        // tied to the embedding table when absent
      // mixed NVFP4 checkpoints hold a feed-forward matrix as weight_packed [n, k / 2] + weight_scale [n, k / 16] (E4M3)
      // + weight_global_scale [1] (+ input_global_scale) instead of weight + weight_scale_inv
      const bool is_weight = s.name.size() > 7 && s.name.compare(s.name.size() - 7, 7, ".weight") == 0;
      const bool is_scale = s.name.size() > 17 && s.name.compare(s.name.size() - 17, 17, ".weight_scale_inv") == 0;
      const std::string stem = is_weight ? s.name.substr(0, s.name.size() - 7) : is_scale ? s.name.substr(0, s.name.size() - 17) : "";
      if (is_scale && stem.compare(0, 4, "mtp.") == 0) {   // a BF16 MTP matrix has no scale grid
        const SafeTensorInfo* wt = model.find(stem + ".weight", &base);
        if (wt && wt->dtype == "BF16") { --rep.expected; continue; }
      }
      const SafeTensorInfo* packed = stem.empty() ? nullptr : model.find(stem + ".weight_packed", &base);
      if (packed && s.kind == QwenLinearKind::Fp8Block128) {
        if (is_scale) continue;                          // accounted for with the weight entry
        const SafeTensorInfo* gs = model.find(stem + ".weight_scale", &base);
        const SafeTensorInfo* gg = model.find(stem + ".weight_global_scale", &base);
        known.insert(stem + ".weight_packed"); known.insert(stem + ".weight_scale");
        known.insert(stem + ".weight_global_scale"); known.insert(stem + ".input_global_scale");
        if (!gs) rep.missing.push_back(stem + ".weight_scale");
        if (!gg) rep.missing.push_back(stem + ".weight_global_scale");
        ++rep.found;
        rep.bytes += packed->nbytes() + (gs ? gs->nbytes() : 0) + (gg ? gg->nbytes() : 0);
        const std::vector<uint64_t> want_p = {s.shape[0], s.shape[1] / 2}, want_s = {s.shape[0], s.shape[1] / 16};
        if (packed->shape != want_p) rep.wrong_shape.push_back(stem + ".weight_packed");
        if (gs && gs->shape != want_s) rep.wrong_shape.push_back(stem + ".weight_scale");
        if (packed->dtype != "U8") rep.wrong_dtype.push_back(stem + ".weight_packed (" + packed->dtype + ", expected U8)");
        if (gs && gs->dtype != "F8_E4M3") rep.wrong_dtype.push_back(stem + ".weight_scale (" + gs->dtype + ", expected F8_E4M3)");
        if (tp_world > 1) {
          const size_t dim = s.rule == QwenShardRule::RowParallel ? 1 : 0;
          if (s.shape[dim] % (uint64_t(tp_world) * 16))
            rep.not_divisible.push_back(stem + ".weight_packed dim " + std::to_string(dim) + " = " + std::to_string(s.shape[dim]));
        }
        continue;
      }
      rep.missing.push_back(s.name);
      continue;
    }
    ++rep.found;
    rep.bytes += info->nbytes();
    if (info->shape != s.shape) rep.wrong_shape.push_back(s.name);
    const bool dtype_ok = s.dtype.find('|') == std::string::npos ? info->dtype == s.dtype
                                                                 : (s.dtype.find(info->dtype) != std::string::npos);
    if (!dtype_ok) rep.wrong_dtype.push_back(s.name + " (" + info->dtype + ", expected " + s.dtype + ")");
    if (tp_world > 1 && s.rule != QwenShardRule::Replicated && s.rule != QwenShardRule::VocabParallel) {
      const size_t dim = s.rule == QwenShardRule::RowParallel ? 1 : 0;
      const uint64_t extent = s.shape.at(std::min(dim, s.shape.size() - 1));
      uint64_t unit = uint64_t(tp_world) * uint64_t(std::max(1, s.group));
      if (s.rule == QwenShardRule::HeadParallel) unit = uint64_t(tp_world);   // checked per q / k / v range by the loader
      const bool scale = s.name.size() > 17 && s.name.compare(s.name.size() - 17, 17, ".weight_scale_inv") == 0;
      if (!scale && extent % unit) rep.not_divisible.push_back(s.name + " dim " + std::to_string(dim) + " = " + std::to_string(extent));
      if (!scale && s.kind == QwenLinearKind::Fp8Block128 && info->dtype == "F8_E4M3" && (extent / uint64_t(tp_world)) % 128)
        rep.not_divisible.push_back(s.name + " shard of " + std::to_string(extent / uint64_t(tp_world)) + " splits a 128-block");
    }
  }
  for (const std::string& n : model.names())
    if (!known.count(n)) rep.unexpected.push_back(n);
  return rep;
}

}  // namespace pocket
