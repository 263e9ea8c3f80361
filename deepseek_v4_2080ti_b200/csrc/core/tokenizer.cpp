#include "tokenizer.hpp"

#include <algorithm>
#include <climits>
#include <stdexcept>

namespace pocket {
namespace {

// GPT-2 byte <-> unicode alphabet: printable bytes map to themselves, the rest to U+0100 + n.
struct ByteAlphabet {
  std::string enc[256];
  std::unordered_map<std::string, uint8_t> dec;
  ByteAlphabet() {
    auto utf8 = [](uint32_t cp) {
      std::string s;
      if (cp < 0x80) s += static_cast<char>(cp);
      else if (cp < 0x800) { s += static_cast<char>(0xC0 | (cp >> 6)); s += static_cast<char>(0x80 | (cp & 0x3F)); }
      else { s += static_cast<char>(0xE0 | (cp >> 12)); s += static_cast<char>(0x80 | ((cp >> 6) & 0x3F)); s += static_cast<char>(0x80 | (cp & 0x3F)); }
      return s;
    };
    int extra = 0;
    for (int b = 0; b < 256; ++b) {
      const bool keep = (b >= 33 && b <= 126) || (b >= 161 && b <= 172) || (b >= 174 && b <= 255);
      enc[b] = utf8(keep ? static_cast<uint32_t>(b) : 256u + static_cast<uint32_t>(extra++));
      dec[enc[b]] = static_cast<uint8_t>(b);
    }
  }
};
const ByteAlphabet& alphabet() { static const ByteAlphabet a; return a; }

size_t utf8_len(unsigned char c) { return c < 0x80 ? 1 : (c >> 5) == 6 ? 2 : (c >> 4) == 14 ? 3 : (c >> 3) == 30 ? 4 : 1; }

}  // namespace

void Tokenizer::build() {
  ids_.clear();
  for (size_t i = 0; i < tokens_.size(); ++i) ids_.emplace(tokens_[i], static_cast<int32_t>(i));
}

Tokenizer Tokenizer::from_vocab(std::vector<std::string> tokens, const std::vector<std::string>& merges, int bos, int eos) {
  Tokenizer t;
  t.tokens_ = std::move(tokens);
  t.bos_ = bos;
  t.eos_ = eos;
  t.build();
  int rank = 0;
  for (const auto& m : merges) t.ranks_.emplace(m, rank++);
  return t;
}

Tokenizer Tokenizer::from_gguf(const GGUFReader& g) {
  const GGUFValue* toks = g.find("tokenizer.ggml.tokens");
  if (!toks || toks->kind != GGUFValue::Kind::Array) throw std::runtime_error("tokenizer: GGUF has no tokenizer.ggml.tokens");
  std::vector<std::string> tokens;
  tokens.reserve(toks->items.size());
  for (const auto& v : toks->items) tokens.push_back(v.s);
  std::vector<std::string> merges;
  if (const GGUFValue* m = g.find("tokenizer.ggml.merges"))
    for (const auto& v : m->items) merges.push_back(v.s);
  Tokenizer t = from_vocab(std::move(tokens), merges, static_cast<int>(g.get_int("tokenizer.ggml.bos_token_id", -1)),
                           static_cast<int>(g.get_int("tokenizer.ggml.eos_token_id", -1)));
  if (const GGUFValue* ty = g.find("tokenizer.ggml.token_type"))
    for (size_t i = 0; i < ty->items.size() && i < t.tokens_.size(); ++i) {
      const int64_t k = ty->items[i].as_int();
      if ((k == 3 || k == 4) && !t.tokens_[i].empty()) t.specials_.push_back(t.tokens_[i]);   // control / user-defined
    }
  std::sort(t.specials_.begin(), t.specials_.end(), [](const std::string& a, const std::string& b) { return a.size() > b.size(); });
  return t;
}

int32_t Tokenizer::find(const std::string& piece) const {
  auto it = ids_.find(piece);
  return it == ids_.end() ? -1 : it->second;
}

void Tokenizer::encode_piece(const std::string& mapped, std::vector<int32_t>& out) const {
  std::vector<std::string> sym;
  for (size_t i = 0; i < mapped.size();) {
    size_t n = utf8_len(static_cast<unsigned char>(mapped[i]));
    sym.push_back(mapped.substr(i, n));
    i += n;
  }
  while (sym.size() > 1) {
    int best = INT_MAX;
    size_t at = 0;
    for (size_t i = 0; i + 1 < sym.size(); ++i) {
      auto it = ranks_.find(sym[i] + " " + sym[i + 1]);
      if (it != ranks_.end() && it->second < best) { best = it->second; at = i; }
    }
    if (best == INT_MAX) break;
    sym[at] += sym[at + 1];
    sym.erase(sym.begin() + static_cast<long>(at) + 1);
  }
  for (const auto& s : sym) {
    int32_t id = find(s);
    if (id >= 0) { out.push_back(id); continue; }
    // unknown multi-character symbol: fall back to its single characters
    for (size_t i = 0; i < s.size();) {
      size_t n = utf8_len(static_cast<unsigned char>(s[i]));
      int32_t cid = find(s.substr(i, n));
      if (cid >= 0) out.push_back(cid);
      i += n;
    }
  }
}

std::vector<int32_t> Tokenizer::encode_basic(const std::string& text, bool add_bos) const {
  std::vector<int32_t> out;
  if (add_bos && bos_ >= 0) out.push_back(bos_);
  const ByteAlphabet& ab = alphabet();
  size_t i = 0;
  std::string piece;
  auto flush = [&] {
    if (piece.empty()) return;
    std::string mapped;
    for (unsigned char c : piece) mapped += ab.enc[c];
    encode_piece(mapped, out);
    piece.clear();
  };
  while (i < text.size()) {
    bool special = false;
    for (const auto& sp : specials_) {
      if (text.compare(i, sp.size(), sp) == 0) {
        flush();
        out.push_back(find(sp));
        i += sp.size();
        special = true;
        break;
      }
    }
    if (special) continue;
    const char c = text[i];
    // a piece is an optional leading space followed by a run of non-space bytes
    if (c == ' ' || c == '\n' || c == '\t' || c == '\r') {
      if (!piece.empty() && !(piece.size() == 1 && piece[0] == ' ' && c != ' ')) flush();
      if (c == ' ') { flush(); piece += c; }
      else { flush(); piece += c; flush(); }
    } else {
      piece += c;
    }
    ++i;
  }
  flush();
  return out;
}

std::string Tokenizer::decode(const std::vector<int32_t>& ids) const {
  const ByteAlphabet& ab = alphabet();
  std::string bytes;
  for (int32_t id : ids) {
    if (id < 0 || static_cast<size_t>(id) >= tokens_.size()) continue;
    const std::string& t = tokens_[static_cast<size_t>(id)];
    if (std::find(specials_.begin(), specials_.end(), t) != specials_.end()) continue;
    for (size_t i = 0; i < t.size();) {
      size_t n = utf8_len(static_cast<unsigned char>(t[i]));
      auto it = ab.dec.find(t.substr(i, n));
      if (it != ab.dec.end()) bytes += static_cast<char>(it->second);
      else bytes += t.substr(i, n);
      i += n;
    }
  }
  return bytes;
}

}  // namespace pocket
