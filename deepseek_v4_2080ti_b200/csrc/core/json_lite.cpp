#include "json_lite.hpp"

#include <cmath>
#include <cstdio>
#include <cstdlib>

namespace pocket {
namespace {

struct Parser {
  const std::string& t;
  size_t p = 0;
  explicit Parser(const std::string& s) : t(s) {}
  [[noreturn]] void fail(const char* what) const {
    throw std::runtime_error(std::string("json: ") + what + " at byte " + std::to_string(p));
  }
  void ws() { while (p < t.size() && (t[p] == ' ' || t[p] == '\n' || t[p] == '\t' || t[p] == '\r')) ++p; }
  bool eat(char c) { ws(); if (p < t.size() && t[p] == c) { ++p; return true; } return false; }
  void expect(char c) { if (!eat(c)) fail("unexpected character"); }

  static void utf8(std::string& out, uint32_t cp) {
    if (cp < 0x80) out += static_cast<char>(cp);
    else if (cp < 0x800) { out += static_cast<char>(0xC0 | (cp >> 6)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
    else if (cp < 0x10000) { out += static_cast<char>(0xE0 | (cp >> 12)); out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
    else { out += static_cast<char>(0xF0 | (cp >> 18)); out += static_cast<char>(0x80 | ((cp >> 12) & 0x3F)); out += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); out += static_cast<char>(0x80 | (cp & 0x3F)); }
  }
  uint32_t hex4() {
    if (p + 4 > t.size()) fail("short \\u escape");
    uint32_t v = 0;
    for (int i = 0; i < 4; ++i) {
      char c = t[p++];
      v <<= 4;
      if (c >= '0' && c <= '9') v |= c - '0';
      else if (c >= 'a' && c <= 'f') v |= c - 'a' + 10;
      else if (c >= 'A' && c <= 'F') v |= c - 'A' + 10;
      else fail("bad hex digit");
    }
    return v;
  }
  std::string str() {
    std::string out;
    for (;;) {
      if (p >= t.size()) fail("unterminated string");
      char c = t[p++];
      if (c == '"') return out;
      if (c != '\\') { out += c; continue; }
      if (p >= t.size()) fail("unterminated escape");
      char e = t[p++];
      switch (e) {
        case '"': out += '"'; break;
        case '\\': out += '\\'; break;
        case '/': out += '/'; break;
        case 'b': out += '\b'; break;
        case 'f': out += '\f'; break;
        case 'n': out += '\n'; break;
        case 'r': out += '\r'; break;
        case 't': out += '\t'; break;
        case 'u': {
          uint32_t cp = hex4();
          if (cp >= 0xD800 && cp <= 0xDBFF && p + 1 < t.size() && t[p] == '\\' && t[p + 1] == 'u') {
            p += 2;
            uint32_t lo = hex4();
            if (lo >= 0xDC00 && lo <= 0xDFFF) cp = 0x10000 + ((cp - 0xD800) << 10) + (lo - 0xDC00);
          }
          utf8(out, cp);
          break;
        }
        default: fail("bad escape");
      }
    }
  }
  Json value(int depth) {
    if (depth > 256) fail("nesting too deep");
    ws();
    if (p >= t.size()) fail("unexpected end");
    char c = t[p];
    if (c == '{') {
      ++p;
      Json o = Json::object();
      if (eat('}')) return o;
      for (;;) {
        ws();
        if (p >= t.size() || t[p] != '"') fail("expected key");
        ++p;
        std::string k = str();
        expect(':');
        o.set(k, value(depth + 1));
        if (eat(',')) continue;
        expect('}');
        return o;
      }
    }
    if (c == '[') {
      ++p;
      Json a = Json::array();
      if (eat(']')) return a;
      for (;;) {
        a.push_back(value(depth + 1));
        if (eat(',')) continue;
        expect(']');
        return a;
      }
    }
    if (c == '"') { ++p; return Json(str()); }
    if (t.compare(p, 4, "true") == 0) { p += 4; return Json(true); }
    if (t.compare(p, 5, "false") == 0) { p += 5; return Json(false); }
    if (t.compare(p, 4, "null") == 0) { p += 4; return Json(); }
    size_t s = p;
    bool is_int = true;
    if (p < t.size() && (t[p] == '-' || t[p] == '+')) ++p;
    while (p < t.size() && ((t[p] >= '0' && t[p] <= '9') || t[p] == '.' || t[p] == 'e' || t[p] == 'E' || t[p] == '-' || t[p] == '+')) {
      if (t[p] == '.' || t[p] == 'e' || t[p] == 'E') is_int = false;
      ++p;
    }
    if (p == s) fail("unexpected token");
    std::string num = t.substr(s, p - s);
    if (is_int) {
      errno = 0;
      char* end = nullptr;
      long long v = std::strtoll(num.c_str(), &end, 10);
      if (errno == 0 && end && *end == 0) return Json(static_cast<int64_t>(v));
    }
    return Json(std::strtod(num.c_str(), nullptr));
  }
};

void dump_to(const Json& j, std::string& out) {
  switch (j.type()) {
    case Json::Type::Null: out += "null"; break;
    case Json::Type::Bool: out += j.as_bool() ? "true" : "false"; break;
    case Json::Type::Number: {
      double d = j.as_double();
      if (std::floor(d) == d && std::fabs(d) < 9e15) out += std::to_string(j.as_int());
      else { char buf[40]; std::snprintf(buf, sizeof buf, "%.17g", d); out += buf; }
      break;
    }
    case Json::Type::String: out += '"'; out += json_escape(j.as_string()); out += '"'; break;
    case Json::Type::Array: {
      out += '[';
      bool first = true;
      for (const auto& v : j.items()) { if (!first) out += ','; first = false; dump_to(v, out); }
      out += ']';
      break;
    }
    case Json::Type::Object: {
      out += '{';
      bool first = true;
      for (const auto& m : j.members()) {
        if (!first) out += ',';
        first = false;
        out += '"'; out += json_escape(m.first); out += "\":";
        dump_to(m.second, out);
      }
      out += '}';
      break;
    }
  }
}

}  // namespace

std::string json_escape(const std::string& s) {
  std::string o;
  o.reserve(s.size() + 8);
  for (unsigned char c : s) {
    switch (c) {
      case '"': o += "\\\""; break;
      case '\\': o += "\\\\"; break;
      case '\n': o += "\\n"; break;
      case '\r': o += "\\r"; break;
      case '\t': o += "\\t"; break;
      default:
        if (c < 0x20) { char b[8]; std::snprintf(b, sizeof b, "\\u%04x", c); o += b; }
        else o += static_cast<char>(c);
    }
  }
  return o;
}

std::string Json::dump() const { std::string s; dump_to(*this, s); return s; }

Json Json::parse(const std::string& text) {
  Parser ps(text);
  Json v = ps.value(0);
  ps.ws();
  if (ps.p != text.size()) ps.fail("trailing characters");
  return v;
}

}  // namespace pocket
