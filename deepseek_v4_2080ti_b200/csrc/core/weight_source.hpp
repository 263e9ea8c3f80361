// Uniform tensor lookup over a Safetensors checkpoint directory or a GGUF file/bundle, with optional
// name mapping (HF module names <-> GGUF "blk.N.*" names) and per-expert slices of stacked GGUF expert
// tensors.  (Role of cpp_engine/include/weight_source.hpp:28-108.)
#pragma once
#include <cstdint>
#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "gguf_reader.hpp"
#include "safetensors_reader.hpp"

namespace pocket {

struct TensorView {
  std::string name;
  std::string dtype;                 // safetensors dtype string, or the ggml type name for GGUF tensors
  uint32_t ggml_type = 0xffffffffu;  // valid for GGUF tensors
  std::vector<uint64_t> shape;       // row-major, outermost first (GGUF shapes are reversed to this order)
  const uint8_t* data = nullptr;
  uint64_t nbytes = 0;
  bool quantized_blocks() const;     // true for GGUF k-/i-quant block formats
};

class WeightSource {
 public:
  static std::unique_ptr<WeightSource> open(const std::string& path);   // directory => safetensors, *.gguf => GGUF
  virtual ~WeightSource() = default;
  virtual std::string format() const = 0;                               // "safetensors" | "gguf"
  virtual std::vector<std::string> names() const = 0;
  virtual bool get(const std::string& name, TensorView& out) = 0;
  // Slice [expert] of a tensor whose outermost dimension enumerates experts (GGUF "…_exps" tensors).
  bool get_expert(const std::string& name, int expert, TensorView& out);
  // Optional translation applied to every requested name before lookup.
  void set_name_map(std::function<std::string(const std::string&)> f) { map_ = std::move(f); }
  virtual const GGUFReader* gguf(size_t shard = 0) const { (void)shard; return nullptr; }

 protected:
  std::string mapped(const std::string& n) const { return map_ ? map_(n) : n; }
  std::function<std::string(const std::string&)> map_;
};

}  // namespace pocket
