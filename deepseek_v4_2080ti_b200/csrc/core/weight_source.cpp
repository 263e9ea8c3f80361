#include "weight_source.hpp"

#include <algorithm>
#include <stdexcept>

#include <sys/stat.h>

namespace pocket {

bool TensorView::quantized_blocks() const {
  if (ggml_type == 0xffffffffu) return false;
  const GGMLTypeInfo* ti = ggml_type_info(ggml_type);
  return ti && ti->block_elems > 1;
}

namespace {

class SafetensorsSource final : public WeightSource {
 public:
  explicit SafetensorsSource(const std::string& dir) : model_(dir) {}
  std::string format() const override { return "safetensors"; }
  std::vector<std::string> names() const override { return model_.names(); }
  bool get(const std::string& name, TensorView& out) override {
    const uint8_t* base = nullptr;
    const SafeTensorInfo* t = model_.find(mapped(name), &base);
    if (!t) return false;
    out.name = t->name;
    out.dtype = t->dtype;
    out.ggml_type = 0xffffffffu;
    out.shape = t->shape;
    out.data = base;
    out.nbytes = t->nbytes();
    return true;
  }

 private:
  SafetensorsModel model_;
};

class GGUFSource final : public WeightSource {
 public:
  explicit GGUFSource(const std::string& path) {
    for (const auto& p : gguf_shard_paths(path)) shards_.push_back(std::make_unique<GGUFReader>(p));
  }
  std::string format() const override { return "gguf"; }
  std::vector<std::string> names() const override {
    std::vector<std::string> out;
    for (const auto& s : shards_)
      for (const auto& t : s->tensors()) out.push_back(t.name);
    return out;
  }
  bool get(const std::string& name, TensorView& out) override {
    const std::string n = mapped(name);
    for (const auto& s : shards_) {
      if (const GGUFTensorInfo* t = s->tensor(n)) {
        out.name = t->name;
        out.ggml_type = t->type;
        const GGMLTypeInfo* ti = ggml_type_info(t->type);
        out.dtype = ti ? ti->name : "unknown";
        out.shape.assign(t->shape.rbegin(), t->shape.rend());
        out.data = s->tensor_data(*t);
        out.nbytes = t->nbytes;
        return true;
      }
    }
    return false;
  }
  const GGUFReader* gguf(size_t shard) const override { return shard < shards_.size() ? shards_[shard].get() : nullptr; }

 private:
  std::vector<std::unique_ptr<GGUFReader>> shards_;
};

}  // namespace

bool WeightSource::get_expert(const std::string& name, int expert, TensorView& out) {
  TensorView full;
  if (!get(name, full)) return false;
  if (full.shape.size() < 2 || expert < 0 || static_cast<uint64_t>(expert) >= full.shape[0]) return false;
  const uint64_t per = full.nbytes / full.shape[0];
  out = full;
  out.shape.erase(out.shape.begin());
  out.data = full.data + per * static_cast<uint64_t>(expert);
  out.nbytes = per;
  out.name = full.name + "[" + std::to_string(expert) + "]";
  return true;
}

std::unique_ptr<WeightSource> WeightSource::open(const std::string& path) {
  struct stat st;
  if (::stat(path.c_str(), &st) != 0) throw std::runtime_error("weight source: no such path " + path);
  if (S_ISDIR(st.st_mode)) return std::make_unique<SafetensorsSource>(path);
  if (path.size() > 5 && path.compare(path.size() - 5, 5, ".gguf") == 0) return std::make_unique<GGUFSource>(path);
  throw std::runtime_error("weight source: expected a checkpoint directory or a .gguf file: " + path);
}

}  // namespace pocket
