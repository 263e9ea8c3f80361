#include "gguf_reader.hpp"

#include <cstdio>
#include <cstring>
#include <stdexcept>

#include <sys/stat.h>

namespace pocket {
namespace {

const GGMLTypeInfo kTypes[] = {
    /* 0*/ {"f32", 1, 4},      {"f16", 1, 2},       {"q4_0", 32, 18},    {"q4_1", 32, 20},   {nullptr, 0, 0},
    /* 5*/ {nullptr, 0, 0},    {"q5_0", 32, 22},    {"q5_1", 32, 24},    {"q8_0", 32, 34},   {"q8_1", 32, 36},
    /*10*/ {"q2_k", 256, 84},  {"q3_k", 256, 110},  {"q4_k", 256, 144},  {"q5_k", 256, 176}, {"q6_k", 256, 210},
    /*15*/ {"q8_k", 256, 292}, {"iq2_xxs", 256, 66}, {"iq2_xs", 256, 74}, {"iq3_xxs", 256, 98}, {"iq1_s", 256, 50},
    /*20*/ {"iq4_nl", 32, 18}, {"iq3_s", 256, 110}, {"iq2_s", 256, 82},  {"iq4_xs", 256, 136}, {"i8", 1, 1},
    /*25*/ {"i16", 1, 2},      {"i32", 1, 4},       {"i64", 1, 8},       {"f64", 1, 8},      {"iq1_m", 256, 56},
    /*30*/ {"bf16", 1, 2},
};

struct Cursor {
  const uint8_t* p;
  const uint8_t* end;
  template <typename T>
  T get() {
    if (static_cast<size_t>(end - p) < sizeof(T)) throw std::runtime_error("gguf: truncated file");
    T v;
    std::memcpy(&v, p, sizeof(T));
    p += sizeof(T);
    return v;
  }
  std::string str() {
    uint64_t n = get<uint64_t>();
    if (n > static_cast<uint64_t>(end - p)) throw std::runtime_error("gguf: string runs past end of file");
    std::string s(reinterpret_cast<const char*>(p), static_cast<size_t>(n));
    p += n;
    return s;
  }
};

GGUFValue read_value(Cursor& c, uint32_t type, int depth = 0) {
  GGUFValue v;
  switch (type) {
    case 0: v.kind = GGUFValue::Kind::UInt; v.u = c.get<uint8_t>(); break;
    case 1: v.kind = GGUFValue::Kind::Int; v.i = c.get<int8_t>(); break;
    case 2: v.kind = GGUFValue::Kind::UInt; v.u = c.get<uint16_t>(); break;
    case 3: v.kind = GGUFValue::Kind::Int; v.i = c.get<int16_t>(); break;
    case 4: v.kind = GGUFValue::Kind::UInt; v.u = c.get<uint32_t>(); break;
    case 5: v.kind = GGUFValue::Kind::Int; v.i = c.get<int32_t>(); break;
    case 6: v.kind = GGUFValue::Kind::Float; v.f = c.get<float>(); break;
    case 7: v.kind = GGUFValue::Kind::Bool; v.b = c.get<uint8_t>() != 0; break;
    case 8: v.kind = GGUFValue::Kind::String; v.s = c.str(); break;
    case 9: {
      if (depth > 2) throw std::runtime_error("gguf: nested arrays too deep");
      v.kind = GGUFValue::Kind::Array;
      v.elem_type = c.get<uint32_t>();
      uint64_t n = c.get<uint64_t>();
      if (n > (1ull << 28)) throw std::runtime_error("gguf: implausible array length");
      v.items.reserve(static_cast<size_t>(n));
      for (uint64_t i = 0; i < n; ++i) v.items.push_back(read_value(c, v.elem_type, depth + 1));
      break;
    }
    case 10: v.kind = GGUFValue::Kind::UInt; v.u = c.get<uint64_t>(); break;
    case 11: v.kind = GGUFValue::Kind::Int; v.i = c.get<int64_t>(); break;
    case 12: v.kind = GGUFValue::Kind::Float; v.f = c.get<double>(); break;
    default: throw std::runtime_error("gguf: unknown metadata type " + std::to_string(type));
  }
  return v;
}

}  // namespace

const GGMLTypeInfo* ggml_type_info(uint32_t type) {
  if (type >= sizeof(kTypes) / sizeof(kTypes[0]) || kTypes[type].name == nullptr) return nullptr;
  return &kTypes[type];
}

GGUFReader::GGUFReader(const std::string& path) : file_(path) {
  Cursor c{file_.data(), file_.data() + file_.size()};
  if (file_.size() < 24 || std::memcmp(c.p, "GGUF", 4) != 0) throw std::runtime_error("gguf: bad magic in " + path);
  c.p += 4;
  version_ = c.get<uint32_t>();
  if (version_ < 2 || version_ > 3) throw std::runtime_error("gguf: unsupported version " + std::to_string(version_));
  const uint64_t n_tensors = c.get<uint64_t>();
  const uint64_t n_kv = c.get<uint64_t>();
  if (n_tensors > (1ull << 24) || n_kv > (1ull << 24)) throw std::runtime_error("gguf: implausible counts");
  for (uint64_t i = 0; i < n_kv; ++i) {
    std::string key = c.str();
    uint32_t type = c.get<uint32_t>();
    kv_[key] = read_value(c, type);
  }
  if (const GGUFValue* a = find("general.alignment")) alignment_ = static_cast<uint64_t>(a->as_int(32));
  if (alignment_ == 0 || (alignment_ & (alignment_ - 1))) throw std::runtime_error("gguf: alignment must be a power of two");
  tensors_.reserve(static_cast<size_t>(n_tensors));
  for (uint64_t i = 0; i < n_tensors; ++i) {
    GGUFTensorInfo t;
    t.name = c.str();
    uint32_t nd = c.get<uint32_t>();
    if (nd > 8) throw std::runtime_error("gguf: too many dimensions in " + t.name);
    for (uint32_t d = 0; d < nd; ++d) t.shape.push_back(c.get<uint64_t>());
    t.type = c.get<uint32_t>();
    t.offset = c.get<uint64_t>();
    const GGMLTypeInfo* ti = ggml_type_info(t.type);
    if (!ti) throw std::runtime_error("gguf: unknown tensor type " + std::to_string(t.type) + " in " + t.name);
    const uint64_t inner = t.shape.empty() ? 1 : t.shape[0];
    if (inner % ti->block_elems) throw std::runtime_error("gguf: row length of " + t.name + " is not a multiple of the block size");
    t.nbytes = t.numel() / ti->block_elems * ti->block_bytes;
    index_[t.name] = tensors_.size();
    tensors_.push_back(std::move(t));
  }
  const uint64_t pos = static_cast<uint64_t>(c.p - file_.data());
  data_offset_ = (pos + alignment_ - 1) / alignment_ * alignment_;
  for (const auto& t : tensors_)
    if (data_offset_ + t.offset + t.nbytes > file_.size())
      throw std::runtime_error("gguf: tensor " + t.name + " runs past end of file");
}

const GGUFValue* GGUFReader::find(const std::string& key) const {
  auto it = kv_.find(key);
  return it == kv_.end() ? nullptr : &it->second;
}
std::string GGUFReader::get_string(const std::string& key, const std::string& dflt) const {
  const GGUFValue* v = find(key);
  return (v && v->kind == GGUFValue::Kind::String) ? v->s : dflt;
}
int64_t GGUFReader::get_int(const std::string& key, int64_t dflt) const {
  const GGUFValue* v = find(key);
  return v ? v->as_int(dflt) : dflt;
}
double GGUFReader::get_float(const std::string& key, double dflt) const {
  const GGUFValue* v = find(key);
  return v ? v->as_float(dflt) : dflt;
}
const GGUFTensorInfo* GGUFReader::tensor(const std::string& name) const {
  auto it = index_.find(name);
  return it == index_.end() ? nullptr : &tensors_[it->second];
}
const uint8_t* GGUFReader::tensor_data(const GGUFTensorInfo& t) const {
  if (data_offset_ + t.offset + t.nbytes > file_.size()) throw std::runtime_error("gguf: tensor data out of range");
  return file_.data() + data_offset_ + t.offset;
}

std::vector<std::string> gguf_shard_paths(const std::string& path) {
  // pattern: <stem>-00001-of-00005.gguf
  const std::string suffix = ".gguf";
  if (path.size() < suffix.size() + 15 || path.compare(path.size() - suffix.size(), suffix.size(), suffix) != 0) return {path};
  const size_t e = path.size() - suffix.size();
  // positions: ...-NNNNN-of-MMMMM
  if (e < 15 || path.compare(e - 9, 4, "-of-") != 0 || path[e - 15] != '-') return {path};
  int total = 0;
  for (size_t i = e - 5; i < e; ++i) { if (path[i] < '0' || path[i] > '9') return {path}; total = total * 10 + (path[i] - '0'); }
  for (size_t i = e - 14; i < e - 9; ++i) if (path[i] < '0' || path[i] > '9') return {path};
  if (total < 1 || total > 99999) return {path};
  std::vector<std::string> out;
  const std::string stem = path.substr(0, e - 15);
  for (int s = 1; s <= total; ++s) {
    char buf[32];
    std::snprintf(buf, sizeof buf, "-%05d-of-%05d", s, total);
    std::string p = stem + buf + suffix;
    struct stat st;
    if (::stat(p.c_str(), &st) != 0) throw std::runtime_error("gguf: missing shard " + p);
    out.push_back(std::move(p));
  }
  return out;
}

}  // namespace pocket
