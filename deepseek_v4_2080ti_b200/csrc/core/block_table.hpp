// Per-slot block rows: a dense [max_slots, max_blocks_per_seq] int32 host image that mirrors the
// device block table the attention kernels read, with dirty-row tracking so only changed rows are
// uploaded.  (Role of cpp_engine/include/block_table.hpp:22-71.)
#pragma once
#include <cstdint>
#include <vector>

#include "block_pool.hpp"

namespace pocket {

class BlockTable {
 public:
  BlockTable(BlockPool& pool, int max_slots, int max_blocks_per_seq);
  int max_slots() const { return max_slots_; }
  int max_blocks_per_seq() const { return max_blocks_; }
  // Grow slot's row so it can hold `tokens` tokens. All-or-nothing; false when the pool is exhausted
  // or the sequence would exceed max_blocks_per_seq.
  bool ensure_capacity(int slot, int64_t tokens);
  // Share the first n blocks of `src` into the (empty) row of `dst` (prefix reuse): refcounts go up.
  bool share_prefix(int dst, int src, int n_blocks);
  // Put `n_blocks` already allocated blocks (held by a prefix cache) at the start of the (empty) row of `dst`; each
  // gains a reference that free_slot gives back.
  bool adopt(int dst, const int32_t* blocks, int n_blocks);
  void free_slot(int slot);
  int blocks_in(int slot) const { return counts_.at(slot); }
  int32_t block_at(int slot, int i) const { return image_[static_cast<size_t>(slot) * max_blocks_ + i]; }
  // Flat KV row index of token position `pos` of `slot`: block * block_tokens + pos % block_tokens.
  int64_t element_offset(int slot, int64_t pos) const;
  const int32_t* image() const { return image_.data(); }
  const int32_t* row(int slot) const { return image_.data() + static_cast<size_t>(slot) * max_blocks_; }
  // Rows changed since the last call; clears the marks.
  std::vector<int> take_dirty_rows();

 private:
  BlockPool& pool_;
  const int max_slots_, max_blocks_;
  std::vector<int32_t> image_;
  std::vector<int> counts_;
  std::vector<uint8_t> dirty_;
};

}  // namespace pocket
