// Byte-level BPE tokenizer built from GGUF metadata (tokenizer.ggml.tokens / merges / token_type,
// bos/eos ids).  encode_basic: split into bytes -> GPT-2 byte alphabet -> greedy lowest-rank merges
// per whitespace-delimited piece; decode is the inverse.  (Role of cpp_engine/include/tokenizer.hpp:13-40.)
#pragma once
#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "gguf_reader.hpp"

namespace pocket {

class Tokenizer {
 public:
  Tokenizer() = default;
  static Tokenizer from_gguf(const GGUFReader& gguf);
  static Tokenizer from_vocab(std::vector<std::string> tokens, const std::vector<std::string>& merges,
                              int bos = -1, int eos = -1);
  size_t vocab_size() const { return tokens_.size(); }
  int bos_id() const { return bos_; }
  int eos_id() const { return eos_; }
  std::vector<int32_t> encode_basic(const std::string& text, bool add_bos = false) const;
  std::string decode(const std::vector<int32_t>& ids) const;
  const std::string& token(int32_t id) const { return tokens_.at(static_cast<size_t>(id)); }
  int32_t find(const std::string& piece) const;   // -1 when absent

 private:
  void build();
  void encode_piece(const std::string& mapped, std::vector<int32_t>& out) const;
  std::vector<std::string> tokens_;
  std::unordered_map<std::string, int32_t> ids_;
  std::unordered_map<std::string, int32_t> ranks_;   // "left right" -> merge rank
  std::vector<std::string> specials_;                // control / user-defined tokens matched verbatim
  int bos_ = -1, eos_ = -1;
};

}  // namespace pocket
