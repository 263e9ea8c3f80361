// GGUF v2/v3 container reader: header, typed metadata, tensor directory, mmap'd tensor data.
// (Role of cpp_engine/include/gguf_reader.hpp + core/gguf_reader.cpp and of the Python reader
// src/loader/gguf/reader.py:121-204; block geometry table from src/loader/gguf/reader.py:27-57.)
#pragma once
#include <cstdint>
#include <map>
#include <string>
#include <vector>

#include "mapped_file.hpp"

namespace pocket {

enum class GGMLType : uint32_t {
  F32 = 0, F16 = 1, Q4_0 = 2, Q4_1 = 3, Q5_0 = 6, Q5_1 = 7, Q8_0 = 8, Q8_1 = 9, Q2_K = 10, Q3_K = 11, Q4_K = 12,
  Q5_K = 13, Q6_K = 14, Q8_K = 15, IQ2_XXS = 16, IQ2_XS = 17, IQ3_XXS = 18, IQ1_S = 19, IQ4_NL = 20, IQ3_S = 21,
  IQ2_S = 22, IQ4_XS = 23, I8 = 24, I16 = 25, I32 = 26, I64 = 27, F64 = 28, IQ1_M = 29, BF16 = 30,
};

struct GGMLTypeInfo { const char* name; uint32_t block_elems; uint32_t block_bytes; };
const GGMLTypeInfo* ggml_type_info(uint32_t type);   // nullptr for unknown ids

struct GGUFValue {
  enum class Kind { None, UInt, Int, Float, Bool, String, Array } kind = Kind::None;
  uint64_t u = 0;
  int64_t i = 0;
  double f = 0;
  bool b = false;
  std::string s;
  uint32_t elem_type = 0;                 // GGUF metadata type id of array elements
  std::vector<GGUFValue> items;           // arrays (strings and scalars)
  int64_t as_int(int64_t d = 0) const { return kind == Kind::UInt ? static_cast<int64_t>(u) : kind == Kind::Int ? i : kind == Kind::Bool ? b : kind == Kind::Float ? static_cast<int64_t>(f) : d; }
  double as_float(double d = 0) const { return kind == Kind::Float ? f : kind == Kind::UInt ? static_cast<double>(u) : kind == Kind::Int ? static_cast<double>(i) : d; }
};

struct GGUFTensorInfo {
  std::string name;
  std::vector<uint64_t> shape;            // GGUF order: shape[0] is the innermost (contiguous) dimension
  uint32_t type = 0;
  uint64_t offset = 0;                    // relative to the data section
  uint64_t nbytes = 0;
  uint64_t numel() const { uint64_t n = 1; for (auto d : shape) n *= d; return n; }
};

class GGUFReader {
 public:
  explicit GGUFReader(const std::string& path);    // throws std::runtime_error on malformed files
  uint32_t version() const { return version_; }
  uint64_t alignment() const { return alignment_; }
  const std::map<std::string, GGUFValue>& metadata() const { return kv_; }
  const GGUFValue* find(const std::string& key) const;
  std::string get_string(const std::string& key, const std::string& dflt = "") const;
  int64_t get_int(const std::string& key, int64_t dflt = 0) const;
  double get_float(const std::string& key, double dflt = 0) const;
  const std::vector<GGUFTensorInfo>& tensors() const { return tensors_; }
  const GGUFTensorInfo* tensor(const std::string& name) const;
  const uint8_t* tensor_data(const GGUFTensorInfo& t) const;      // pointer into the mapping (bounds checked)
  const std::string& path() const { return file_.path(); }
  uint64_t data_offset() const { return data_offset_; }

 private:
  MappedFile file_;
  uint32_t version_ = 0;
  uint64_t alignment_ = 32, data_offset_ = 0;
  std::map<std::string, GGUFValue> kv_;
  std::vector<GGUFTensorInfo> tensors_;
  std::map<std::string, size_t> index_;
};

// Multi-shard bundles "name-00001-of-0000N.gguf": returns all shard paths (or {path} for single files).
std::vector<std::string> gguf_shard_paths(const std::string& first_or_any_shard);

}  // namespace pocket
