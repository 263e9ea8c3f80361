#include "safetensors_reader.hpp"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>
#include <stdexcept>

#include <dirent.h>
#include <sys/stat.h>

#include "json_lite.hpp"

namespace pocket {

int safetensors_dtype_size(const std::string& d) {
  if (d == "F8_E4M3" || d == "F8_E5M2" || d == "F8_E8M0" || d == "U8" || d == "I8" || d == "BOOL") return 1;
  if (d == "BF16" || d == "F16" || d == "I16" || d == "U16") return 2;
  if (d == "F32" || d == "I32" || d == "U32") return 4;
  if (d == "F64" || d == "I64" || d == "U64") return 8;
  return 0;
}

SafetensorsFile::SafetensorsFile(const std::string& path) : file_(path) {
  if (file_.size() < 8) throw std::runtime_error("safetensors: file too small: " + path);
  uint64_t hlen = 0;
  std::memcpy(&hlen, file_.data(), 8);
  if (hlen == 0 || hlen > file_.size() - 8 || hlen > (1ull << 30)) throw std::runtime_error("safetensors: bad header length in " + path);
  payload_ = 8 + hlen;
  Json header = Json::parse(std::string(reinterpret_cast<const char*>(file_.data() + 8), static_cast<size_t>(hlen)));
  if (!header.is_object()) throw std::runtime_error("safetensors: header is not an object");
  const uint64_t payload_size = file_.size() - payload_;
  for (const auto& m : header.members()) {
    if (m.first == "__metadata__") {
      for (const auto& kv : m.second.members()) meta_[kv.first] = kv.second.as_string();
      continue;
    }
    SafeTensorInfo t;
    t.name = m.first;
    t.dtype = m.second["dtype"].as_string();
    for (const auto& d : m.second["shape"].items()) t.shape.push_back(static_cast<uint64_t>(d.as_int()));
    const Json& off = m.second["data_offsets"];
    if (off.size() != 2) throw std::runtime_error("safetensors: bad data_offsets for " + t.name);
    t.begin = static_cast<uint64_t>(off[0].as_int());
    t.end = static_cast<uint64_t>(off[1].as_int());
    const int es = safetensors_dtype_size(t.dtype);
    if (t.end < t.begin || t.end > payload_size) throw std::runtime_error("safetensors: tensor " + t.name + " out of range");
    if (es && t.numel() * es != t.nbytes()) throw std::runtime_error("safetensors: size mismatch for " + t.name);
    index_[t.name] = tensors_.size();
    tensors_.push_back(std::move(t));
  }
}

const SafeTensorInfo* SafetensorsFile::find(const std::string& name) const {
  auto it = index_.find(name);
  return it == index_.end() ? nullptr : &tensors_[it->second];
}

static bool exists(const std::string& p) {
  struct stat st;
  return ::stat(p.c_str(), &st) == 0;
}

SafetensorsModel::SafetensorsModel(const std::string& dir) : dir_(dir) {
  const std::string idx = dir + "/model.safetensors.index.json";
  if (exists(idx)) {
    std::ifstream f(idx);
    std::stringstream ss;
    ss << f.rdbuf();
    Json j = Json::parse(ss.str());
    for (const auto& m : j["weight_map"].members()) {
      where_[m.first] = m.second.as_string();
      if (std::find(shard_files_.begin(), shard_files_.end(), m.second.as_string()) == shard_files_.end())
        shard_files_.push_back(m.second.as_string());
    }
    if (where_.empty()) throw std::runtime_error("safetensors: empty weight_map in " + idx);
    return;
  }
  // no index: every *.safetensors file in the directory
  DIR* d = ::opendir(dir.c_str());
  if (!d) throw std::runtime_error("safetensors: cannot open directory " + dir);
  while (dirent* e = ::readdir(d)) {
    std::string n = e->d_name;
    if (n.size() > 12 && n.compare(n.size() - 12, 12, ".safetensors") == 0) shard_files_.push_back(n);
  }
  ::closedir(d);
  std::sort(shard_files_.begin(), shard_files_.end());
  if (shard_files_.empty()) throw std::runtime_error("safetensors: no .safetensors files in " + dir);
  for (const auto& f : shard_files_)
    for (const auto& t : shard(f).tensors()) where_[t.name] = f;
}

SafetensorsFile& SafetensorsModel::shard(const std::string& file) {
  auto it = open_.find(file);
  if (it == open_.end()) it = open_.emplace(file, std::make_unique<SafetensorsFile>(dir_ + "/" + file)).first;
  return *it->second;
}

std::vector<std::string> SafetensorsModel::names() const {
  std::vector<std::string> out;
  out.reserve(where_.size());
  for (const auto& kv : where_) out.push_back(kv.first);
  return out;
}

const SafeTensorInfo* SafetensorsModel::find(const std::string& name, const uint8_t** base) {
  auto it = where_.find(name);
  if (it == where_.end()) return nullptr;
  SafetensorsFile& f = shard(it->second);
  const SafeTensorInfo* t = f.find(name);
  if (t && base) *base = f.data(*t);
  return t;
}

}  // namespace pocket
