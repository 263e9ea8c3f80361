// Safetensors reader: 8-byte little-endian header length, JSON header, mmap'd payload; plus the
// sharded-checkpoint index (model.safetensors.index.json -> tensor name -> shard file).
// (Role of cpp_engine/include/safetensors_reader.hpp, safetensors_model.hpp.)
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "mapped_file.hpp"

namespace pocket {

struct SafeTensorInfo {
  std::string name;
  std::string dtype;                 // F8_E4M3, F8_E5M2, BF16, F16, F32, U8, I8, I32, I64, F8_E8M0, ...
  std::vector<uint64_t> shape;
  uint64_t begin = 0, end = 0;       // byte range inside the payload
  uint64_t nbytes() const { return end - begin; }
  uint64_t numel() const { uint64_t n = 1; for (auto d : shape) n *= d; return n; }
};

int safetensors_dtype_size(const std::string& dtype);   // bytes per element, 0 if unknown

class SafetensorsFile {
 public:
  explicit SafetensorsFile(const std::string& path);
  const std::vector<SafeTensorInfo>& tensors() const { return tensors_; }
  const SafeTensorInfo* find(const std::string& name) const;
  const uint8_t* data(const SafeTensorInfo& t) const { return file_.data() + payload_ + t.begin; }
  const std::map<std::string, std::string>& metadata() const { return meta_; }
  const std::string& path() const { return file_.path(); }

 private:
  MappedFile file_;
  uint64_t payload_ = 0;
  std::vector<SafeTensorInfo> tensors_;
  std::map<std::string, size_t> index_;
  std::map<std::string, std::string> meta_;
};

// A checkpoint directory: either a single model.safetensors or an index + shards. Shards are mapped lazily.
class SafetensorsModel {
 public:
  explicit SafetensorsModel(const std::string& dir);
  std::vector<std::string> names() const;
  bool contains(const std::string& name) const { return where_.count(name) != 0; }
  // Returns the tensor's info and sets *base to its first byte (valid while this object lives).
  const SafeTensorInfo* find(const std::string& name, const uint8_t** base);
  const std::string& dir() const { return dir_; }
  size_t shard_count() const { return shard_files_.size(); }

 private:
  SafetensorsFile& shard(const std::string& file);
  std::string dir_;
  std::map<std::string, std::string> where_;                    // tensor -> shard file name
  std::vector<std::string> shard_files_;
  std::map<std::string, std::unique_ptr<SafetensorsFile>> open_;
};

}  // namespace pocket
