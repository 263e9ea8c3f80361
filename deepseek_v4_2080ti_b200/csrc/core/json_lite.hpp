// Minimal JSON value + recursive-descent parser + serializer (no third-party dependency).
// Same role as the reference's cpp_engine/include/json_lite.hpp; this one keeps object key
// order and parses numbers as double with an "is integer" flag.
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

namespace pocket {

class Json {
 public:
  enum class Type { Null, Bool, Number, String, Array, Object };
  using Array = std::vector<Json>;
  using Member = std::pair<std::string, Json>;
  using Object = std::vector<Member>;

  Json() = default;
  Json(std::nullptr_t) {}
  Json(bool b) : type_(Type::Bool), b_(b) {}
  Json(double d) : type_(Type::Number), n_(d) {}
  Json(int64_t i) : type_(Type::Number), n_(static_cast<double>(i)), is_int_(true), i_(i) {}
  Json(int i) : Json(static_cast<int64_t>(i)) {}
  Json(const char* s) : type_(Type::String), s_(s) {}
  Json(std::string s) : type_(Type::String), s_(std::move(s)) {}
  static Json array() { Json j; j.type_ = Type::Array; return j; }
  static Json object() { Json j; j.type_ = Type::Object; return j; }

  Type type() const { return type_; }
  bool is_null() const { return type_ == Type::Null; }
  bool is_bool() const { return type_ == Type::Bool; }
  bool is_number() const { return type_ == Type::Number; }
  bool is_string() const { return type_ == Type::String; }
  bool is_array() const { return type_ == Type::Array; }
  bool is_object() const { return type_ == Type::Object; }

  bool as_bool(bool dflt = false) const { return is_bool() ? b_ : dflt; }
  double as_double(double dflt = 0) const { return is_number() ? n_ : dflt; }
  int64_t as_int(int64_t dflt = 0) const { return is_number() ? (is_int_ ? i_ : static_cast<int64_t>(n_)) : dflt; }
  const std::string& as_string() const { static const std::string e; return is_string() ? s_ : e; }
  const Array& items() const { static const Array e; return is_array() ? a_ : e; }
  const Object& members() const { static const Object e; return is_object() ? o_ : e; }

  bool contains(const std::string& k) const { return find(k) != nullptr; }
  const Json* find(const std::string& k) const {
    if (!is_object()) return nullptr;
    for (const auto& m : o_) if (m.first == k) return &m.second;
    return nullptr;
  }
  const Json& operator[](const std::string& k) const { static const Json n; const Json* p = find(k); return p ? *p : n; }
  const Json& operator[](size_t i) const { static const Json n; return (is_array() && i < a_.size()) ? a_[i] : n; }
  size_t size() const { return is_array() ? a_.size() : is_object() ? o_.size() : 0; }

  void push_back(Json v) { type_ = Type::Array; a_.push_back(std::move(v)); }
  void set(const std::string& k, Json v) {
    type_ = Type::Object;
    for (auto& m : o_) if (m.first == k) { m.second = std::move(v); return; }
    o_.emplace_back(k, std::move(v));
  }

  std::string dump() const;
  static Json parse(const std::string& text);   // throws std::runtime_error with byte offset on error

 private:
  Type type_ = Type::Null;
  bool b_ = false;
  double n_ = 0;
  bool is_int_ = false;
  int64_t i_ = 0;
  std::string s_;
  Array a_;
  Object o_;
};

std::string json_escape(const std::string& s);

}  // namespace pocket
