// Native engine for the Qwen-style hybrid model: checkpoint -> device weights, paged KV / recurrent state,
// prefill and batched decode over the kernel library's C interface.
#include "qwen_engine.hpp"

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>

#include "../kernels/ops.h"

namespace pocket {

namespace {
constexpr int kHead = 128;          // head width of both attention kinds (the kernels are specialised for it)
constexpr int kStreamMaxT = 32;     // largest batch the weight-streaming decode GEMM serves
constexpr int kSMs = 148;

double now_s() {
  return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

size_t dtype_size(const std::string& d) {
  if (d == "BF16" || d == "F16") return 2;
  if (d == "F32" || d == "I32") return 4;
  if (d == "F8_E4M3" || d == "U8" || d == "I8") return 1;
  throw std::runtime_error("unsupported checkpoint dtype " + d);
}

TensorView need(WeightSource& ws, const std::string& name) {
  TensorView v;
  if (!ws.get(name, v)) throw std::runtime_error("checkpoint lacks tensor " + name);
  return v;
}

// Split count for the tile-decoding GEMM at small T (same rule as the Python front end: the split count that
// wastes least of the last wave, at least 8 k-blocks per split).
int pick_splits(int t, int n, int k) {
  if (t > 128) return 1;
  const int bn = t <= 16 ? 16 : t <= 32 ? 32 : t <= 64 ? 64 : 128;
  const int tiles = ((n + 127) / 128) * ((t + bn - 1) / bn);
  const int kb = (k + 63) / 64;
  const int max_s = std::max(1, std::min(kb / 8, t <= 16 ? 16 : t <= 64 ? 8 : 4));
  int best = 1;
  double best_eff = 0;
  for (int s = 1; s <= max_s; ++s) {
    const int per = (kb + s - 1) / s;
    if ((kb + per - 1) / per != s) continue;
    const int waves = (tiles * s + kSMs - 1) / kSMs;
    const double eff = double(tiles) * kb / (double(waves) * kSMs * per);
    if (eff > best_eff + 0.02) { best = s; best_eff = eff; }
  }
  return best;
}

// Split count for the weight-streaming GEMM: smallest count that fills 85% of the waves.
int pick_splits_stream(int n, int k) {
  const int tiles = (n + 127) / 128, kblk = k / 128;
  int best = 1;
  double best_eff = 0;
  for (int s = 1; s <= std::max(1, std::min(kblk / 4, 16)); ++s) {
    const int per = (kblk + s - 1) / s;
    if ((kblk + per - 1) / per != s) continue;
    const int waves = (tiles * s + kSMs - 1) / kSMs;
    const double eff = double(tiles) * kblk / (double(waves) * kSMs * per);
    if (eff > best_eff + 0.05) { best = s; best_eff = eff; }
    if (best_eff >= 0.85) break;
  }
  return best;
}
}  // namespace

// Activation and workspace buffers, sized once for the prefill chunk and the decode batch.
struct QwenNativeEngine::Scratch {
  int rows = 0;                       // capacity in token rows
  DeviceBuffer ids, pos, kv_slots, meta, slot_ids, kv_len, bt_batch;
  DeviceBuffer h, x, d_attn, d_mlp, proj, mixed, core, y, ab, g, beta, q, gate, attn, gu, act;
  DeviceBuffer logits, next_idx, next_val, status, merge;
  DeviceBuffer gdn_ws, splitk_ws, counters, dec_ws;
  DeviceBuffer xq, inv_c, xq2, inv_c2;
  size_t splitk_floats = 0;
  std::vector<int32_t> host_i32;
};

void QwenNativeEngine::rc(int code, const char* what, int launches) {
  if (code != 0) throw std::runtime_error(std::string("kernel launch failed: ") + what + " rc=" + std::to_string(code));
  stats_.kernel_launches += launches;
}

void QwenNativeEngine::check_status(const char* where) {
  int st = 0;
  cuda_check(cudaMemcpyAsync(&st, s_->status.get(), sizeof(int), cudaMemcpyDeviceToHost, stream_), "status readback");
  cuda_check(cudaStreamSynchronize(stream_), where);
  if (st != 0) {
    cudaMemsetAsync(s_->status.get(), 0, sizeof(int), stream_);
    throw std::runtime_error(std::string(where) + ": a kernel reported status " + std::to_string(st) +
                             " (a bounded wait ran out or an argument check failed)");
  }
}

QwenNativeEngine::QwenNativeEngine(const QwenConfig& cfg, WeightSource& weights, const QwenEngineOptions& opt)
    : cfg_(cfg), opt_(opt) {
  rng_.seed(opt.seed);
  cfg_.validate(1);
  if (cfg_.head_dim != kHead || cfg_.linear_key_head_dim != kHead || cfg_.linear_value_head_dim != kHead)
    throw std::runtime_error("the attention kernels are built for 128-wide heads");
  cuda_check(cudaSetDevice(opt_.device), "cudaSetDevice");
  cuda_check(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking), "cudaStreamCreate");
  n_layers_ = opt_.layers > 0 ? std::min<int>(opt_.layers, cfg_.num_hidden_layers) : int(cfg_.num_hidden_layers);
  const int W = std::max(1, opt_.tp_world), tp_r = opt_.tp_rank;
  if (W > 1) {
    if (cfg_.num_attention_heads % W || cfg_.num_key_value_heads % W || cfg_.linear_num_value_heads % W ||
        cfg_.linear_num_key_heads % W || (cfg_.intermediate_size / W) % 128 || cfg_.intermediate_size % W)
      throw std::runtime_error("head counts / feed-forward width do not divide over " + std::to_string(W) + " ranks");
    if (opt_.sampling.temperature > 0.f)
      throw std::runtime_error("the native engine samples on the host from full logits: multi-rank runs are greedy");
    tp_.init(W, tp_r, opt_.device, opt_.nccl_id_path);
  }
  hq_ = int(cfg_.num_attention_heads) / W; hkv_ = int(cfg_.num_key_value_heads) / W;
  hv_ = int(cfg_.linear_num_value_heads) / W; hk_ = int(cfg_.linear_num_key_heads) / W;
  kd_ = hk_ * kHead; vd_ = hv_ * kHead; cw_ = 2 * kd_ + vd_;
  inter_ = int(cfg_.intermediate_size) / W;
  const int vper = (int(cfg_.vocab_size) + W - 1) / W;
  vocab_lo_ = tp_r * vper;
  vocab_n_ = std::max(0, std::min(int(cfg_.vocab_size), vocab_lo_ + vper) - vocab_lo_);
  rot_ = int(cfg_.rotary_dim());

  const double t0 = now_s();
  load(weights);
  cuda_check(cudaStreamSynchronize(stream_), "weight load");
  stats_.load_seconds = now_s() - t0;

  // ---- KV cache, recurrent state, block table
  const int bs = opt_.block_tokens;
  max_blocks_per_seq_ = int((opt_.max_context + bs - 1) / bs);
  if (opt_.prefix_cache_interval < 0 || opt_.prefix_cache_interval % bs)
    throw std::runtime_error("prefix_cache_interval must be a multiple of block_tokens");
  num_blocks_ = max_blocks_per_seq_ * opt_.max_slots + 1;          // block 0 is the scratch block
  // cached prefixes keep their blocks after the sequence that wrote them is gone: room for one context per entry
  // (entries are dropped, oldest first, when a running sequence needs the blocks)
  if (opt_.prefix_cache_interval > 0) num_blocks_ += max_blocks_per_seq_ * std::max(1, opt_.prefix_cache_entries);
  pool_ = std::make_unique<BlockPool>(num_blocks_, bs);
  table_ = std::make_unique<BlockTable>(*pool_, opt_.max_slots, max_blocks_per_seq_);
  lengths_.assign(opt_.max_slots, 0);
  slot_used_.assign(opt_.max_slots, 0);
  kv_layer_stride_ = size_t(num_blocks_) * hkv_ * bs * kHead;      // elements per full-attention layer
  const int kw = int(cfg_.linear_conv_kernel_dim);
  state_layer_stride_ = size_t(hv_) * kHead * kHead;
  state_slot_stride_ = state_layer_stride_ * std::max(1, n_lin_);
  tail_layer_stride_ = size_t(kw - 1) * cw_;
  tail_slot_stride_ = tail_layer_stride_ * std::max(1, n_lin_);
  k_cache_.reset(std::max<size_t>(1, n_full_) * kv_layer_stride_ * 2, true);
  v_cache_.reset(std::max<size_t>(1, n_full_) * kv_layer_stride_ * 2, true);
  states_.reset(state_slot_stride_ * opt_.max_slots * sizeof(float), true);
  tails_.reset(tail_slot_stride_ * opt_.max_slots * 2, true);
  block_table_dev_.reset(size_t(opt_.max_slots) * max_blocks_per_seq_ * sizeof(int32_t), true);
  stats_.state_bytes = k_cache_.bytes() + v_cache_.bytes() + states_.bytes() + tails_.bytes();

  std::vector<float> inv(rot_ / 2);
  for (int i = 0; i < rot_ / 2; ++i) inv[i] = float(1.0 / std::pow(cfg_.rope_theta, double(2 * i) / rot_));
  inv_freq_.reset(std::max<size_t>(4, inv.size() * sizeof(float)));
  if (!inv.empty()) cuda_check(cudaMemcpy(inv_freq_.get(), inv.data(), inv.size() * 4, cudaMemcpyHostToDevice), "inv_freq");

  // ---- scratch
  s_ = std::make_unique<Scratch>();
  Scratch& s = *s_;
  const size_t R = size_t(std::max(opt_.prefill_chunk, kStreamMaxT));
  s.rows = int(R);
  const size_t H = size_t(cfg_.hidden_size), I = size_t(inter_), V = size_t(vocab_n_);
  const size_t gate_mul = cfg_.attn_output_gate ? 2 : 1;
  const size_t proj_w = std::max<size_t>(size_t(cw_) + vd_, (size_t(hq_) * gate_mul + 2 * hkv_) * kHead);
  s.ids.reset(R * 4); s.pos.reset(R * 4); s.kv_slots.reset(R * 4); s.meta.reset(64);
  s.slot_ids.reset(64 * 4); s.kv_len.reset(64 * 4); s.bt_batch.reset(size_t(64) * max_blocks_per_seq_ * 4, true);
  s.h.reset(R * H * 2); s.x.reset(R * H * 2); s.d_attn.reset(R * H * 2); s.d_mlp.reset(R * H * 2);
  s.proj.reset(R * proj_w * 2); s.mixed.reset(R * cw_ * 2); s.core.reset(R * vd_ * 2); s.y.reset(R * vd_ * 2);
  s.ab.reset(R * 2 * hv_ * 2 + 64); s.g.reset(R * hv_ * 4 + 64); s.beta.reset(R * hv_ * 4 + 64);
  s.q.reset(R * hq_ * kHead * 2); s.gate.reset(R * hq_ * kHead * 2); s.attn.reset(R * hq_ * kHead * 2);
  s.gu.reset(R * 2 * I * 2); s.act.reset(R * I * 2);
  s.logits.reset(size_t(opt_.max_slots > 64 ? opt_.max_slots : 64) * V * 4);
  s.next_idx.reset(64 * 4); s.next_val.reset(64 * 4); s.status.reset(4, true);
  s.merge.reset(size_t(W) * 64 * 8);
  s.gdn_ws.reset(size_t(std::max<long long>(1, b200_gdn_workspace_floats(int(R), std::max(1, hv_)))) * 4);
  s.splitk_floats = size_t(1) << 24;
  s.splitk_ws.reset(s.splitk_floats * 4);
  s.counters.reset(size_t(1 << 16) * 4, true);
  s.dec_ws.reset(size_t(64) * hq_ * 64 * (kHead + 2) * 4);
  const size_t maxk = std::max({H, I, size_t(vd_), size_t(hq_) * kHead});
  s.xq.reset(size_t(kStreamMaxT) * 3 * maxk); s.inv_c.reset(64 * 4);
  s.xq2.reset(size_t(kStreamMaxT) * 3 * maxk); s.inv_c2.reset(64 * 4);

  // the fused decode path needs every FP8 reduction width to be a multiple of the 128-wide scale block
  stream_ok_ = (H % 128 == 0) && (I % 128 == 0) && (vd_ % 128 == 0) && ((hq_ * kHead) % 128 == 0) && kw == 4 && hk_ > 0 &&
               (hv_ / hk_ == 1 || hv_ / hk_ == 2 || hv_ / hk_ == 4);
}

QwenNativeEngine::~QwenNativeEngine() {
  if (stream_) { cudaStreamSynchronize(stream_); cudaStreamDestroy(stream_); }
}

// ------------------------------------------------------------------------------------------------ loading
DeviceBuffer QwenNativeEngine::load_vector(WeightSource& ws, const std::string& name, bool to_f32, long long first,
                                           long long count) {
  TensorView v = need(ws, name);
  size_t total = 1;
  for (auto d : v.shape) total *= d;
  const size_t esz = dtype_size(v.dtype);
  if (count < 0) count = (long long)total - first;
  if (first < 0 || size_t(first + count) > total) throw std::runtime_error(name + ": shard outside the tensor");
  const size_t nbytes = size_t(count) * esz;
  DeviceBuffer raw(nbytes);
  cuda_check(cudaMemcpyAsync(raw.get(), reinterpret_cast<const uint8_t*>(v.data) + size_t(first) * esz, nbytes,
                             cudaMemcpyHostToDevice, stream_), name.c_str());
  stats_.weight_bytes += nbytes;
  if (!to_f32) {
    if (v.dtype != "BF16") throw std::runtime_error(name + ": expected BF16, found " + v.dtype);
    cuda_check(cudaStreamSynchronize(stream_), name.c_str());
    return raw;
  }
  if (v.dtype == "F32") { cuda_check(cudaStreamSynchronize(stream_), name.c_str()); return raw; }
  if (v.dtype != "BF16") throw std::runtime_error(name + ": expected BF16 or F32, found " + v.dtype);
  DeviceBuffer out(size_t(count) * 4);
  rc(b200_bf16_to_f32(raw.get(), out.as<float>(), count, stream_), "bf16_to_f32");
  cuda_check(cudaStreamSynchronize(stream_), name.c_str());
  return out;
}

// Compact device copy of the window [row0, row0+rows) x [col0, col0+cols) of a row-major host matrix.
DeviceBuffer QwenNativeEngine::upload_window(const TensorView& v, size_t elem, long long row0, long long rows,
                                             long long col0, long long cols) {
  const size_t pitch = size_t(v.shape[1]) * elem;
  DeviceBuffer out(size_t(rows) * cols * elem);
  const uint8_t* src = reinterpret_cast<const uint8_t*>(v.data) + size_t(row0) * pitch + size_t(col0) * elem;
  cuda_check(cudaMemcpy2DAsync(out.get(), size_t(cols) * elem, src, pitch, size_t(cols) * elem, size_t(rows),
                               cudaMemcpyHostToDevice, stream_), "window upload");
  return out;
}

PackedMatrix QwenNativeEngine::load_bf16(WeightSource& ws, const std::vector<Piece>& pieces) {
  PackedMatrix m;
  m.wfmt = 0;
  struct Part { TensorView v; long long r0, rows; };
  std::vector<Part> parts;
  for (auto& pc : pieces) {
    TensorView v = need(ws, pc.name);
    if (v.dtype != "BF16" || v.shape.size() != 2) throw std::runtime_error(pc.name + ": expected a BF16 matrix");
    if (pc.col0 != 0 || pc.cols >= 0) throw std::runtime_error(pc.name + ": bf16 matrices are sharded by rows only");
    const long long rows = pc.rows < 0 ? (long long)v.shape[0] - pc.row0 : pc.rows;
    if (pc.row0 < 0 || pc.row0 + rows > (long long)v.shape[0]) throw std::runtime_error(pc.name + ": row shard outside the matrix");
    if (m.k && int(v.shape[1]) != m.k) throw std::runtime_error(pc.name + ": inner widths differ");
    m.k = int(v.shape[1]);
    m.n += int(rows);
    parts.push_back({v, pc.row0, rows});
  }
  m.weight.reset(std::max<size_t>(2, size_t(m.n) * m.k * 2));
  size_t off = 0;
  for (auto& p : parts) {
    const size_t nb = size_t(p.rows) * m.k * 2;
    cuda_check(cudaMemcpyAsync(m.weight.as<uint8_t>() + off, reinterpret_cast<const uint8_t*>(p.v.data) + size_t(p.r0) * m.k * 2,
                               nb, cudaMemcpyHostToDevice, stream_), "bf16 upload");
    off += nb;
  }
  cuda_check(cudaStreamSynchronize(stream_), "bf16 upload");
  stats_.weight_bytes += off;
  return m;
}

PackedMatrix QwenNativeEngine::load_fp8(WeightSource& ws, const std::vector<Piece>& pieces) {
  PackedMatrix m;
  m.wfmt = 1;
  struct Part { TensorView w, s; long long r0, rows, c0, cols; };
  std::vector<Part> parts;
  for (auto& pc : pieces) {
    Part p{need(ws, pc.name + ".weight"), need(ws, pc.name + ".weight_scale_inv"), pc.row0, pc.rows, pc.col0, pc.cols};
    if (p.w.dtype != "F8_E4M3" || p.w.shape.size() != 2) throw std::runtime_error(pc.name + ": expected an F8_E4M3 matrix");
    if (p.rows < 0) p.rows = (long long)p.w.shape[0] - p.r0;
    if (p.cols < 0) p.cols = (long long)p.w.shape[1] - p.c0;
    if (p.r0 < 0 || p.c0 < 0 || p.r0 + p.rows > (long long)p.w.shape[0] || p.c0 + p.cols > (long long)p.w.shape[1])
      throw std::runtime_error(pc.name + ": shard outside the matrix");
    const bool whole = p.r0 == 0 && p.c0 == 0 && p.rows == (long long)p.w.shape[0] && p.cols == (long long)p.w.shape[1];
    if (!whole && (p.r0 % 128 || p.c0 % 128 || (p.rows % 128 && p.r0 + p.rows != (long long)p.w.shape[0]) ||
                   (p.cols % 128 && p.c0 + p.cols != (long long)p.w.shape[1])))
      throw std::runtime_error(pc.name + ": an FP8 shard must keep whole 128 x 128 scale blocks");
    if (m.k && int(p.cols) != m.k) throw std::runtime_error(pc.name + ": inner widths differ");
    m.k = int(p.cols);
    if (pieces.size() > 1 && p.rows % 128) throw std::runtime_error(pc.name + ": fused projections need 128-row multiples");
    m.n += int(p.rows);
    parts.push_back(p);
  }
  const int kb_total = (m.k + 63) / 64, sld = (m.k + 127) / 128;
  m.weight.reset(b200_prepack_fp8_bytes(m.n, m.k));
  m.scales.reset(size_t((m.n + 127) / 128) * sld * 4);
  int row = 0;
  for (auto& p : parts) {
    const int n = int(p.rows);
    const size_t ssz = dtype_size(p.s.dtype);
    const long long srows = (p.rows + 127) / 128;
    DeviceBuffer raw = upload_window(p.w, 1, p.r0, p.rows, p.c0, p.cols);
    DeviceBuffer sraw = upload_window(p.s, ssz, p.r0 / 128, srows, p.c0 / 128, sld);
    rc(b200_prepack_fp8(raw.get(), m.weight.as<uint8_t>() + size_t(row / 128) * kb_total * 8192, n, m.k, stream_), "prepack_fp8");
    const size_t sc = size_t(srows) * sld;
    float* dst = m.scales.as<float>() + size_t(row / 128) * sld;
    if (p.s.dtype == "F32") {
      cuda_check(cudaMemcpyAsync(dst, sraw.get(), sc * 4, cudaMemcpyDeviceToDevice, stream_), "scale copy");
    } else if (p.s.dtype == "BF16") {
      rc(b200_bf16_to_f32(sraw.get(), dst, (long long)sc, stream_), "bf16_to_f32");
    } else {
      throw std::runtime_error("scale tensor dtype " + p.s.dtype + " is not supported");
    }
    cuda_check(cudaStreamSynchronize(stream_), "fp8 prepack");   // raw buffers die at scope end
    stats_.weight_bytes += size_t(p.rows) * p.cols + sc * 4;
    row += n;
  }
  return m;
}

void QwenNativeEngine::load(WeightSource& ws) {
  const std::string root = "model.language_model.";
  const int W = std::max(1, opt_.tp_world), R = opt_.tp_rank;
  {
    // the embedding table is replicated (1.5 GB at the 27B shape): the lookup then needs no collective
    TensorView e = need(ws, root + "embed_tokens.weight");
    if (e.dtype != "BF16") throw std::runtime_error("embedding table must be BF16");
    embed_.reset(e.nbytes);
    cuda_check(cudaMemcpyAsync(embed_.get(), e.data, e.nbytes, cudaMemcpyHostToDevice, stream_), "embed upload");
    stats_.weight_bytes += e.nbytes;
  }
  final_norm_ = load_vector(ws, root + "norm.weight", false);
  TensorView probe;
  lm_head_ = load_bf16(ws, {{ws.get("lm_head.weight", probe) ? "lm_head.weight" : root + "embed_tokens.weight",
                             vocab_lo_, vocab_n_}});
  const long long I = cfg_.intermediate_size, Il = inter_;
  const long long kd_full = (long long)cfg_.linear_num_key_heads * kHead, vd_full = (long long)cfg_.linear_num_value_heads * kHead;
  const int gate_mul = cfg_.attn_output_gate ? 2 : 1;
  const long long qrows = (long long)hq_ * kHead * gate_mul, kvrows = (long long)hkv_ * kHead;
  (void)I; (void)W;
  layers_.resize(n_layers_);
  for (int i = 0; i < n_layers_; ++i) {
    QwenLayer& L = layers_[i];
    const std::string p = root + "layers." + std::to_string(i) + ".";
    L.linear = cfg_.layer_types.at(i) == "linear_attention";
    L.in_ln = load_vector(ws, p + "input_layernorm.weight", false);
    L.post_ln = load_vector(ws, p + "post_attention_layernorm.weight", false);
    L.gate_up = load_fp8(ws, {{p + "mlp.gate_proj", R * Il, Il}, {p + "mlp.up_proj", R * Il, Il}});
    L.down = load_fp8(ws, {{p + "mlp.down_proj", 0, -1, R * Il, Il}});
    if (L.linear) {
      const std::string a = p + "linear_attn.";
      // in_proj_qkv holds q | k | v row blocks: each block is split over the ranks, like the conv channels
      L.proj = load_fp8(ws, {{a + "in_proj_qkv", R * (long long)kd_, kd_}, {a + "in_proj_qkv", kd_full + R * (long long)kd_, kd_},
                             {a + "in_proj_qkv", 2 * kd_full + R * (long long)vd_, vd_}, {a + "in_proj_z", R * (long long)vd_, vd_}});
      L.out = load_fp8(ws, {{a + "out_proj", 0, -1, R * (long long)vd_, vd_}});
      L.ab = load_bf16(ws, {{a + "in_proj_a.weight", R * (long long)hv_, hv_}, {a + "in_proj_b.weight", R * (long long)hv_, hv_}});
      {
        // conv1d.weight [2kd + vd, 1, kw]: the same three channel blocks
        TensorView cv = need(ws, a + "conv1d.weight");
        if (cv.dtype != "BF16") throw std::runtime_error("conv1d.weight must be BF16");
        const size_t kwb = size_t(cfg_.linear_conv_kernel_dim) * 2;
        L.conv_w.reset(size_t(cw_) * kwb);
        const long long blk[3][2] = {{R * (long long)kd_, kd_}, {kd_full + R * (long long)kd_, kd_}, {2 * kd_full + R * (long long)vd_, vd_}};
        size_t off = 0;
        for (auto& b : blk) {
          cuda_check(cudaMemcpyAsync(L.conv_w.as<uint8_t>() + off, reinterpret_cast<const uint8_t*>(cv.data) + size_t(b[0]) * kwb,
                                     size_t(b[1]) * kwb, cudaMemcpyHostToDevice, stream_), "conv upload");
          off += size_t(b[1]) * kwb;
        }
        cuda_check(cudaStreamSynchronize(stream_), "conv upload");
        stats_.weight_bytes += off;
        (void)vd_full;
      }
      L.a_log = load_vector(ws, a + "A_log", true, R * (long long)hv_, hv_);
      L.dt_bias = load_vector(ws, a + "dt_bias", true, R * (long long)hv_, hv_);
      L.gdn_norm = load_vector(ws, a + "norm.weight", false);
      L.cache_index = n_lin_++;
    } else {
      const std::string a = p + "self_attn.";
      L.proj = load_fp8(ws, {{a + "q_proj", R * qrows, qrows}, {a + "k_proj", R * kvrows, kvrows}, {a + "v_proj", R * kvrows, kvrows}});
      L.out = load_fp8(ws, {{a + "o_proj", 0, -1, R * (long long)hq_ * kHead, (long long)hq_ * kHead}});
      L.q_norm = load_vector(ws, a + "q_norm.weight", false);
      L.k_norm = load_vector(ws, a + "k_norm.weight", false);
      L.cache_index = n_full_++;
    }
  }
}

// Row-parallel outputs: sum over the ranks (bf16, in place; NCCL on the engine's stream).
void QwenNativeEngine::reduce_rows(void* buf, int T) {
  if (tp_.active()) tp_.all_reduce_bf16(buf, size_t(T) * size_t(cfg_.hidden_size), stream_);
}

// ------------------------------------------------------------------------------------------------ slots
int QwenNativeEngine::allocate_slot() {
  for (int s = 0; s < opt_.max_slots; ++s) {
    if (slot_used_[s]) continue;
    slot_used_[s] = 1;
    lengths_[s] = 0;
    cuda_check(cudaMemsetAsync(states_.as<float>() + state_slot_stride_ * s, 0, state_slot_stride_ * 4, stream_), "state clear");
    cuda_check(cudaMemsetAsync(tails_.as<uint8_t>() + tail_slot_stride_ * s * 2, 0, tail_slot_stride_ * 2, stream_), "tail clear");
    return s;
  }
  return -1;
}

void QwenNativeEngine::free_slot(int slot) {
  if (slot < 0 || slot >= opt_.max_slots || !slot_used_[slot]) return;
  table_->free_slot(slot);
  slot_used_[slot] = 0;
  lengths_[slot] = 0;
}

bool QwenNativeEngine::reserve(int slot, int64_t tokens) {
  if (tokens > opt_.max_context) return false;
  return table_->ensure_capacity(slot, tokens);
}

void QwenNativeEngine::upload_block_rows() {
  for (int r : table_->take_dirty_rows())
    cuda_check(cudaMemcpyAsync(block_table_dev_.as<int32_t>() + size_t(r) * max_blocks_per_seq_, table_->row(r),
                               size_t(max_blocks_per_seq_) * 4, cudaMemcpyHostToDevice, stream_), "block table upload");
}

bool QwenNativeEngine::is_eos(int32_t token) const {
  return std::find(opt_.eos_tokens.begin(), opt_.eos_tokens.end(), token) != opt_.eos_tokens.end();
}

// ------------------------------------------------------------------------------------------------ projections
QwenTargetHead QwenNativeEngine::target_head() const {
  QwenTargetHead h;
  h.wfmt = lm_head_.wfmt;
  h.weight = lm_head_.weight.get();
  h.scales = lm_head_.scales.as<float>();
  h.local_vocab = lm_head_.n;
  h.hidden = lm_head_.k;
  h.vocab_start = vocab_lo_;
  h.status = s_->status.as<int>();
  return h;
}

void QwenNativeEngine::linear(const void* x, const PackedMatrix& w, void* out, int T, float* out_f32) {
  Scratch& s = *s_;
  if (out_f32) {
    rc(b200_gemm_wdec_ex(w.wfmt, w.weight.get(), w.scales.as<float>(), x, nullptr, out_f32, nullptr, T, w.n, w.k, 1,
                         nullptr, s.status.as<int>(), stream_), "gemm(f32)");
    return;
  }
  int splits = pick_splits(T, w.n, w.k);
  while (splits > 1 && size_t(splits) * T * w.n > s.splitk_floats) --splits;
  const int bn = b200_gemm_pick_bn(T);
  if (splits > 1 && size_t((w.n + 127) / 128) * ((T + bn - 1) / bn) > (1u << 16)) splits = 1;
  rc(b200_gemm_wdec_ex(w.wfmt, w.weight.get(), w.scales.as<float>(), x, out, splits > 1 ? s.splitk_ws.as<float>() : nullptr,
                       nullptr, T, w.n, w.k, splits, s.counters.as<int>(), s.status.as<int>(), stream_), "gemm");
}

void QwenNativeEngine::linear_stream(const void* xq, const float* inv_c, const PackedMatrix& w, void* out, int T) {
  Scratch& s = *s_;
  int splits = pick_splits_stream(w.n, w.k);
  while (splits > 1 && size_t(splits) * T * w.n > s.splitk_floats) --splits;
  rc(b200_gemm_w8a8s(w.weight.get(), w.scales.as<float>(), xq, inv_c, out, nullptr, T, w.n, w.k, splits,
                     s.splitk_ws.as<float>(), s.counters.as<int>(), s.status.as<int>(), stream_), "gemm_stream");
}

// ------------------------------------------------------------------------------------------------ prefill
int32_t QwenNativeEngine::forward_prefill(int slot, const int32_t* tokens, int T, int64_t pos0, bool want_token) {
  Scratch& s = *s_;
  if (T > s.rows) throw std::runtime_error("prefill chunk exceeds the scratch capacity");
  const int bs = opt_.block_tokens, H = int(cfg_.hidden_size), I = inter_;
  const float eps = float(cfg_.rms_norm_eps);
  upload_block_rows();
  std::vector<int32_t>& hb = s.host_i32;
  hb.resize(size_t(T) * 2 + 3);
  for (int i = 0; i < T; ++i) {
    const int64_t p = pos0 + i;
    hb[i] = int32_t(p);
    hb[T + i] = int32_t(table_->element_offset(slot, p));
  }
  hb[2 * T] = 0; hb[2 * T + 1] = T; hb[2 * T + 2] = int32_t(pos0 + T);
  cuda_check(cudaMemcpyAsync(s.ids.get(), tokens, size_t(T) * 4, cudaMemcpyHostToDevice, stream_), "ids");
  cuda_check(cudaMemcpyAsync(s.pos.get(), hb.data(), size_t(T) * 4, cudaMemcpyHostToDevice, stream_), "pos");
  cuda_check(cudaMemcpyAsync(s.kv_slots.get(), hb.data() + T, size_t(T) * 4, cudaMemcpyHostToDevice, stream_), "kv slots");
  cuda_check(cudaMemcpyAsync(s.meta.get(), hb.data() + 2 * T, 12, cudaMemcpyHostToDevice, stream_), "meta");
  const int* meta = s.meta.as<int>();
  const int* bt_row = block_table_dev_.as<int32_t>() + size_t(slot) * max_blocks_per_seq_;

  rc(b200_embedding(s.ids.as<int>(), embed_.get(), s.h.get(), T, H, 0, int(cfg_.vocab_size), stream_), "embedding");
  const void* delta = nullptr;
  for (int li = 0; li < n_layers_; ++li) {
    QwenLayer& L = layers_[li];
    rc(b200_rmsnorm(s.h.get(), delta, nullptr, 0, L.in_ln.get(), s.x.get(), T, H, eps, 1, delta ? 1 : 0, stream_), "rmsnorm");
    linear(s.x.get(), L.proj, s.proj.get(), T);
    const int ldp = L.proj.n;
    if (L.linear) {
      linear(s.x.get(), L.ab, s.ab.get(), T);
      rc(b200_gdn_gates(s.ab.get(), 2 * hv_, 0, hv_, L.a_log.as<float>(), L.dt_bias.as<float>(), s.g.as<float>(),
                        s.beta.as<float>(), T, hv_, stream_), "gdn_gates");
      void* tail = tails_.as<uint8_t>() + (tail_slot_stride_ * slot + tail_layer_stride_ * L.cache_index) * 2;
      float* state = states_.as<float>() + state_slot_stride_ * slot + state_layer_stride_ * L.cache_index;
      rc(b200_conv_silu(s.proj.get(), ldp, L.conv_w.get(), tail, s.mixed.get(), cw_, T, cw_,
                        int(cfg_.linear_conv_kernel_dim), 1, stream_), "conv_silu");
      rc(b200_gdn_chunked(s.mixed.get(), cw_, 0, kd_, 2 * kd_, s.g.as<float>(), s.beta.as<float>(), state, s.core.get(),
                          s.gdn_ws.as<float>(), T, hv_, hk_, stream_), "gdn_chunked", 2);
      rc(b200_gated_rmsnorm(s.core.get(), s.proj.as<uint8_t>() + size_t(cw_) * 2, L.gdn_norm.get(), s.y.get(),
                            (long long)T * hv_, kHead, eps, hv_, ldp, stream_), "gated_rmsnorm");
      linear(s.y.get(), L.out, s.d_attn.get(), T);
      reduce_rows(s.d_attn.get(), T);
    } else {
      const int gate_mul = cfg_.attn_output_gate ? 2 : 1;
      const int qw = hq_ * kHead * gate_mul;
      uint8_t* kc = k_cache_.as<uint8_t>() + kv_layer_stride_ * L.cache_index * 2;
      uint8_t* vc = v_cache_.as<uint8_t>() + kv_layer_stride_ * L.cache_index * 2;
      rc(b200_qk_norm_rope_append(s.proj.get(), ldp, 0, kHead * gate_mul, cfg_.attn_output_gate ? 1 : 0, s.proj.get(), ldp,
                                  qw, s.proj.get(), ldp, qw + hkv_ * kHead, L.q_norm.get(), L.k_norm.get(), 1, eps,
                                  inv_freq_.as<float>(), rot_, 1.0f, s.pos.as<int>(), s.kv_slots.as<int>(), s.q.get(),
                                  cfg_.attn_output_gate ? s.gate.get() : nullptr, kc, vc, bs, T, hq_, hkv_, stream_),
         "qk_norm_rope_append");
      rc(b200_gqa_prefill(s.q.get(), kc, vc, s.attn.get(), cfg_.attn_output_gate ? s.gate.get() : nullptr, bt_row, meta,
                          meta + 1, meta + 2, 1, T, T, max_blocks_per_seq_, num_blocks_, bs, hq_, hkv_,
                          1.0f / std::sqrt(float(kHead)), s.status.as<int>(), stream_), "gqa_prefill");
      linear(s.attn.get(), L.out, s.d_attn.get(), T);
      reduce_rows(s.d_attn.get(), T);
    }
    rc(b200_rmsnorm(s.h.get(), s.d_attn.get(), nullptr, 0, L.post_ln.get(), s.x.get(), T, H, eps, 1, 1, stream_), "rmsnorm");
    linear(s.x.get(), L.gate_up, s.gu.get(), T);
    rc(b200_silu_mul(s.gu.get(), s.act.get(), T, I, stream_), "silu_mul");
    linear(s.act.get(), L.down, s.d_mlp.get(), T);
    reduce_rows(s.d_mlp.get(), T);
    delta = s.d_mlp.get();
  }
  lengths_[slot] = pos0 + T;
  if (!want_token) { check_status("prefill"); return -1; }
  // final norm + head on the last row only
  uint8_t* last = s.h.as<uint8_t>() + size_t(T - 1) * H * 2;
  const uint8_t* dlast = delta ? reinterpret_cast<const uint8_t*>(delta) + size_t(T - 1) * H * 2 : nullptr;
  rc(b200_rmsnorm(last, dlast, nullptr, 0, final_norm_.get(), s.x.get(), 1, H, eps, 1, dlast ? 1 : 0, stream_), "final norm");
  rc(target_head().project(s.x.get(), s.logits.as<float>(), 1, stream_), "lm_head");
  rc(b200_argmax(s.logits.get(), 1, vocab_n_, vocab_n_, 1, vocab_lo_, s.next_idx.as<int>(), s.next_val.as<float>(), stream_),
     "argmax", 2);
  int32_t tok = -1;
  if (tp_.active()) {
    tok = tp_.argmax_merge(s.next_val.as<float>(), s.next_idx.as<int32_t>(), 1, s.merge.get(), stream_).at(0);
  } else {
    cuda_check(cudaMemcpyAsync(&tok, s.next_idx.get(), 4, cudaMemcpyDeviceToHost, stream_), "token readback");
  }
  check_status("prefill");
  if (opt_.sampling.temperature > 0.f) sample_rows(1, &tok);
  return tok;
}

// ------------------------------------------------------------------------------------------------ decode
void QwenNativeEngine::forward_decode(const std::vector<int>& slots, const std::vector<int32_t>& tokens,
                                      std::vector<int32_t>& next) {
  Scratch& s = *s_;
  const int B = int(slots.size());
  if (B <= 0 || B > 64 || B > s.rows) throw std::runtime_error("decode batch must hold 1..64 sequences");
  const int bs = opt_.block_tokens, H = int(cfg_.hidden_size), I = inter_, V = vocab_n_;
  const float eps = float(cfg_.rms_norm_eps);
  for (int i = 0; i < B; ++i)
    if (!reserve(slots[i], lengths_.at(slots[i]) + 1)) throw std::runtime_error("KV cache exhausted");
  upload_block_rows();
  std::vector<int32_t>& hb = s.host_i32;
  hb.assign(size_t(B) * 5, 0);
  int64_t max_kv = 1;
  for (int i = 0; i < B; ++i) {
    const int64_t p = lengths_[slots[i]];
    hb[i] = tokens[i];
    hb[B + i] = int32_t(p);
    hb[2 * B + i] = int32_t(table_->element_offset(slots[i], p));
    hb[3 * B + i] = slots[i];
    hb[4 * B + i] = int32_t(p + 1);
    max_kv = std::max<int64_t>(max_kv, p + 1);
    cuda_check(cudaMemcpyAsync(s.bt_batch.as<int32_t>() + size_t(i) * max_blocks_per_seq_, table_->row(slots[i]),
                               size_t(max_blocks_per_seq_) * 4, cudaMemcpyHostToDevice, stream_), "batch block rows");
  }
  cuda_check(cudaMemcpyAsync(s.ids.get(), hb.data(), size_t(B) * 4, cudaMemcpyHostToDevice, stream_), "ids");
  cuda_check(cudaMemcpyAsync(s.pos.get(), hb.data() + B, size_t(B) * 4, cudaMemcpyHostToDevice, stream_), "pos");
  cuda_check(cudaMemcpyAsync(s.kv_slots.get(), hb.data() + 2 * B, size_t(B) * 4, cudaMemcpyHostToDevice, stream_), "kv slots");
  cuda_check(cudaMemcpyAsync(s.slot_ids.get(), hb.data() + 3 * B, size_t(B) * 4, cudaMemcpyHostToDevice, stream_), "slot ids");
  cuda_check(cudaMemcpyAsync(s.kv_len.get(), hb.data() + 4 * B, size_t(B) * 4, cudaMemcpyHostToDevice, stream_), "kv len");

  const bool fused = stream_ok_ && B <= kStreamMaxT;
  int terms = 2;
  if (fused) b200_gemm_w8a8s_layout(B, &terms);
  const int att_splits = int(std::max<int64_t>(1, std::min<int64_t>({64, (2 * kSMs) / std::max(1, B * hkv_), (max_kv + 255) / 256})));
  const float scale = 1.0f / std::sqrt(float(kHead));
  const int gate_mul = cfg_.attn_output_gate ? 2 : 1;
  const int qw = hq_ * kHead * gate_mul;
  const int kw = int(cfg_.linear_conv_kernel_dim);

  rc(b200_embedding(s.ids.as<int>(), embed_.get(), s.h.get(), B, H, 0, int(cfg_.vocab_size), stream_), "embedding");
  const void* delta = nullptr;
  for (int li = 0; li < n_layers_; ++li) {
    QwenLayer& L = layers_[li];
    const int ldp = L.proj.n;
    void* tails = tails_.as<uint8_t>() + tail_layer_stride_ * L.cache_index * 2;
    float* states = states_.as<float>() + state_layer_stride_ * L.cache_index;
    uint8_t* kc = k_cache_.as<uint8_t>() + kv_layer_stride_ * L.cache_index * 2;
    uint8_t* vc = v_cache_.as<uint8_t>() + kv_layer_stride_ * L.cache_index * 2;
    if (fused) {
      rc(b200_rmsnorm_split(s.h.get(), delta, L.in_ln.get(), L.linear ? s.x.get() : nullptr, s.xq.get(), s.inv_c.as<float>(),
                            B, H, eps, 1, terms, stream_), "rmsnorm_split");
      linear_stream(s.xq.get(), s.inv_c.as<float>(), L.proj, s.proj.get(), B);
    } else {
      rc(b200_rmsnorm(s.h.get(), delta, nullptr, 0, L.in_ln.get(), s.x.get(), B, H, eps, 1, delta ? 1 : 0, stream_), "rmsnorm");
      linear(s.x.get(), L.proj, s.proj.get(), B);
    }
    const void* mix_out = nullptr;      // [B, K of the output projection]
    if (L.linear) {
      if (fused) {
        rc(b200_gdn_decode_fused(s.proj.get(), ldp, s.x.get(), H, L.ab.weight.get(), L.a_log.as<float>(),
                                 L.dt_bias.as<float>(), L.conv_w.get(), kw, tails, (long long)tail_slot_stride_, states,
                                 (long long)state_slot_stride_, s.slot_ids.as<int>(), L.gdn_norm.get(), s.y.get(), B, hv_,
                                 hk_, eps, stream_), "gdn_decode_fused");
      } else {
        linear(s.x.get(), L.ab, s.ab.get(), B);
        rc(b200_gdn_gates(s.ab.get(), 2 * hv_, 0, hv_, L.a_log.as<float>(), L.dt_bias.as<float>(), s.g.as<float>(),
                          s.beta.as<float>(), B, hv_, stream_), "gdn_gates");
        rc(b200_conv_silu_step(s.proj.get(), ldp, L.conv_w.get(), tails, (long long)tail_slot_stride_, s.slot_ids.as<int>(),
                               s.mixed.get(), cw_, B, cw_, kw, stream_), "conv_silu_step");
        rc(b200_gdn_step(states, (long long)state_slot_stride_, s.slot_ids.as<int>(), s.mixed.get(), cw_, 0, kd_, 2 * kd_,
                         s.g.as<float>(), s.beta.as<float>(), s.core.get(), B, hv_, hk_, stream_), "gdn_step");
        rc(b200_gated_rmsnorm(s.core.get(), s.proj.as<uint8_t>() + size_t(cw_) * 2, L.gdn_norm.get(), s.y.get(),
                              (long long)B * hv_, kHead, eps, hv_, ldp, stream_), "gated_rmsnorm");
      }
      mix_out = s.y.get();
    } else {
      rc(b200_qk_norm_rope_append(s.proj.get(), ldp, 0, kHead * gate_mul, cfg_.attn_output_gate ? 1 : 0, s.proj.get(), ldp,
                                  qw, s.proj.get(), ldp, qw + hkv_ * kHead, L.q_norm.get(), L.k_norm.get(), 1, eps,
                                  inv_freq_.as<float>(), rot_, 1.0f, s.pos.as<int>(), s.kv_slots.as<int>(), s.q.get(),
                                  cfg_.attn_output_gate ? s.gate.get() : nullptr, kc, vc, bs, B, hq_, hkv_, stream_),
         "qk_norm_rope_append");
      rc(b200_gqa_decode(s.q.get(), kc, vc, s.attn.get(), cfg_.attn_output_gate ? s.gate.get() : nullptr,
                         s.bt_batch.as<int>(), s.kv_len.as<int>(), s.dec_ws.as<float>(), B, max_blocks_per_seq_, bs, hq_,
                         hkv_, att_splits, scale, stream_), "gqa_decode", att_splits > 1 ? 2 : 1);
      mix_out = s.attn.get();
    }
    if (fused) {
      rc(b200_act_split_e4m3(mix_out, B, L.out.k, terms, s.xq2.get(), s.inv_c2.as<float>(), stream_), "act_split");
      linear_stream(s.xq2.get(), s.inv_c2.as<float>(), L.out, s.d_attn.get(), B);
      reduce_rows(s.d_attn.get(), B);
      rc(b200_rmsnorm_split(s.h.get(), s.d_attn.get(), L.post_ln.get(), nullptr, s.xq.get(), s.inv_c.as<float>(), B, H, eps,
                            1, terms, stream_), "rmsnorm_split");
      linear_stream(s.xq.get(), s.inv_c.as<float>(), L.gate_up, s.gu.get(), B);
      rc(b200_silu_mul_split(s.gu.get(), s.xq2.get(), s.inv_c2.as<float>(), B, I, terms, stream_), "silu_mul_split");
      linear_stream(s.xq2.get(), s.inv_c2.as<float>(), L.down, s.d_mlp.get(), B);
    } else {
      linear(mix_out, L.out, s.d_attn.get(), B);
      reduce_rows(s.d_attn.get(), B);
      rc(b200_rmsnorm(s.h.get(), s.d_attn.get(), nullptr, 0, L.post_ln.get(), s.x.get(), B, H, eps, 1, 1, stream_), "rmsnorm");
      linear(s.x.get(), L.gate_up, s.gu.get(), B);
      rc(b200_silu_mul(s.gu.get(), s.act.get(), B, I, stream_), "silu_mul");
      linear(s.act.get(), L.down, s.d_mlp.get(), B);
    }
    reduce_rows(s.d_mlp.get(), B);
    delta = s.d_mlp.get();
  }
  rc(b200_rmsnorm(s.h.get(), delta, nullptr, 0, final_norm_.get(), s.x.get(), B, H, eps, 1, delta ? 1 : 0, stream_), "final norm");
  rc(target_head().project(s.x.get(), s.logits.as<float>(), B, stream_), "lm_head");
  rc(b200_argmax(s.logits.get(), 1, V, V, B, vocab_lo_, s.next_idx.as<int>(), s.next_val.as<float>(), stream_), "argmax", 2);
  next.resize(B);
  if (tp_.active()) {
    next = tp_.argmax_merge(s.next_val.as<float>(), s.next_idx.as<int32_t>(), B, s.merge.get(), stream_);
  } else {
    cuda_check(cudaMemcpyAsync(next.data(), s.next_idx.get(), size_t(B) * 4, cudaMemcpyDeviceToHost, stream_), "token readback");
  }
  check_status("decode");
  if (opt_.sampling.temperature > 0.f) sample_rows(B, next.data());
  for (int i = 0; i < B; ++i) lengths_[slots[i]] += 1;
}

// Temperature / top-k / top-p sampling on the host from the fp32 logits of the last forward.
void QwenNativeEngine::sample_rows(int rows, int32_t* tokens) {
  const size_t V = size_t(cfg_.vocab_size);
  host_logits_.resize(size_t(rows) * V);
  cuda_check(cudaMemcpy(host_logits_.data(), s_->logits.get(), host_logits_.size() * 4, cudaMemcpyDeviceToHost), "logits readback");
  for (int r = 0; r < rows; ++r) tokens[r] = sample(host_logits_.data() + size_t(r) * V, int(V), opt_.sampling, rng_);
}

// ------------------------------------------------------------------------------------------------ batch interface
// ------------------------------------------------------------------------------------------------ prefix cache
int64_t QwenNativeEngine::prefix_lookup(int slot, const std::vector<int32_t>& tokens) {
  PrefixEntry* best = nullptr;
  for (auto& e : prefix_) {
    const size_t n = e->tokens.size();
    if (n + 1 > tokens.size() || (best && n <= best->tokens.size())) continue;     // at least one token stays to compute
    if (std::equal(e->tokens.begin(), e->tokens.end(), tokens.begin())) best = e.get();
  }
  if (!best) return 0;
  if (!table_->adopt(slot, best->blocks.data(), int(best->blocks.size()))) return 0;
  cuda_check(cudaMemcpyAsync(states_.as<float>() + state_slot_stride_ * slot, best->states.get(), state_slot_stride_ * 4,
                             cudaMemcpyDeviceToDevice, stream_), "prefix state restore");
  cuda_check(cudaMemcpyAsync(tails_.as<uint8_t>() + tail_slot_stride_ * slot * 2, best->tails.get(), tail_slot_stride_ * 2,
                             cudaMemcpyDeviceToDevice, stream_), "prefix tail restore");
  best->stamp = ++prefix_clock_;
  lengths_[slot] = int64_t(best->tokens.size());
  ++stats_.prefix_hits;
  stats_.prefix_tokens_reused += best->tokens.size();
  return lengths_[slot];
}

void QwenNativeEngine::prefix_drop(size_t i) {
  for (int32_t b : prefix_[i]->blocks) pool_->release(b);
  prefix_.erase(prefix_.begin() + long(i));
  ++stats_.prefix_evictions;
}

void QwenNativeEngine::prefix_store(int slot, const int32_t* tokens, int64_t n) {
  for (auto& e : prefix_)
    if (int64_t(e->tokens.size()) == n && std::equal(e->tokens.begin(), e->tokens.end(), tokens)) {
      e->stamp = ++prefix_clock_;
      return;
    }
  while (int(prefix_.size()) >= std::max(1, opt_.prefix_cache_entries)) {
    size_t oldest = 0;
    for (size_t i = 1; i < prefix_.size(); ++i)
      if (prefix_[i]->stamp < prefix_[oldest]->stamp) oldest = i;
    prefix_drop(oldest);
  }
  auto e = std::make_unique<PrefixEntry>();
  e->tokens.assign(tokens, tokens + n);
  const int nb = int(n / opt_.block_tokens);
  for (int i = 0; i < nb; ++i) {
    const int32_t b = table_->block_at(slot, i);
    pool_->retain(b);
    e->blocks.push_back(b);
  }
  e->states = DeviceBuffer(state_slot_stride_ * 4);
  e->tails = DeviceBuffer(tail_slot_stride_ * 2);
  cuda_check(cudaMemcpyAsync(e->states.get(), states_.as<float>() + state_slot_stride_ * slot, state_slot_stride_ * 4,
                             cudaMemcpyDeviceToDevice, stream_), "prefix state snapshot");
  cuda_check(cudaMemcpyAsync(e->tails.get(), tails_.as<uint8_t>() + tail_slot_stride_ * slot * 2, tail_slot_stride_ * 2,
                             cudaMemcpyDeviceToDevice, stream_), "prefix tail snapshot");
  e->stamp = ++prefix_clock_;
  prefix_.push_back(std::move(e));
  ++stats_.prefix_snapshots;
}

StepResult QwenNativeEngine::batch_prefill(const std::vector<PrefillItem>& items) {
  StepResult r;
  const int64_t every = opt_.prefix_cache_interval;
  for (const PrefillItem& it : items) {
    if (it.tokens.empty()) { r.next_tokens.push_back(-1); continue; }
    if (it.position != lengths_.at(it.slot)) throw std::runtime_error("prefill position does not continue the slot");
    int32_t tok = -1;
    const int total = int(it.tokens.size());
    int o = 0;
    // a fresh sequence may resume from a cached prefix; snapshots are taken only for prompts that arrive whole
    // (position 0 and last_chunk), so a stored prefix is always a prefix of a complete prompt
    const bool cacheable = every > 0 && it.position == 0 && it.last_chunk;
    if (cacheable) o = int(prefix_lookup(it.slot, it.tokens));
    while (o < total) {
      int t = std::min(opt_.prefill_chunk, total - o);
      if (cacheable) {
        const int64_t boundary = (int64_t(o) / every + 1) * every;              // next snapshot point after o
        if (boundary < total) t = int(std::min<int64_t>(t, boundary - o));
      }
      while (!reserve(it.slot, it.position + o + t)) {
        if (prefix_.empty() || it.position + o + t > opt_.max_context) throw std::runtime_error("KV cache exhausted");
        size_t oldest = 0;                                  // cached prefixes give way to running sequences
        for (size_t i = 1; i < prefix_.size(); ++i)
          if (prefix_[i]->stamp < prefix_[oldest]->stamp) oldest = i;
        prefix_drop(oldest);
      }
      const bool last = it.last_chunk && o + t >= total;
      tok = forward_prefill(it.slot, it.tokens.data() + o, t, it.position + o, last);
      o += t;
      if (cacheable && o < total && o % every == 0) prefix_store(it.slot, it.tokens.data(), o);
    }
    r.next_tokens.push_back(tok);
  }
  return r;
}

StepResult QwenNativeEngine::batch_decode(const std::vector<int>& slots, const std::vector<int32_t>& tokens) {
  StepResult r;
  forward_decode(slots, tokens, r.next_tokens);
  return r;
}

std::vector<int32_t> QwenNativeEngine::generate(const std::vector<int32_t>& prompt, int max_new_tokens, double* prefill_s,
                                                double* decode_s) {
  const int slot = allocate_slot();
  if (slot < 0) throw std::runtime_error("no free slot");
  std::vector<int32_t> out;
  try {
    double t0 = now_s();
    PrefillItem it;
    it.slot = slot; it.tokens = prompt; it.position = 0; it.last_chunk = true;
    int32_t tok = batch_prefill({it}).next_tokens.at(0);
    if (prefill_s) *prefill_s = now_s() - t0;
    t0 = now_s();
    out.push_back(tok);
    while (int(out.size()) < max_new_tokens && !is_eos(tok) && lengths_[slot] + 1 <= opt_.max_context) {
      tok = batch_decode({slot}, {tok}).next_tokens.at(0);
      out.push_back(tok);
    }
    if (decode_s) *decode_s = now_s() - t0;
  } catch (...) {
    free_slot(slot);
    throw;
  }
  free_slot(slot);
  return out;
}

std::vector<std::pair<int32_t, float>> QwenNativeEngine::last_topk(int k) {
  // multi-rank: this rank's vocabulary shard only (ids are global)
  const size_t V = size_t(vocab_n_);
  std::vector<float> row(V);
  cuda_check(cudaMemcpy(row.data(), s_->logits.get(), V * 4, cudaMemcpyDeviceToHost), "logits readback");
  std::vector<int32_t> idx(V);
  for (size_t i = 0; i < V; ++i) idx[i] = int32_t(i);
  k = int(std::min<size_t>(size_t(std::max(1, k)), V));
  std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), [&](int32_t a, int32_t b) { return row[a] > row[b] || (row[a] == row[b] && a < b); });
  std::vector<std::pair<int32_t, float>> out;
  for (int i = 0; i < k; ++i) out.emplace_back(idx[i] + vocab_lo_, row[idx[i]]);
  return out;
}

}  // namespace pocket
