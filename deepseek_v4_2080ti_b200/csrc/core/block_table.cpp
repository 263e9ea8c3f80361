#include "block_table.hpp"

#include <stdexcept>

namespace pocket {

BlockTable::BlockTable(BlockPool& pool, int max_slots, int max_blocks_per_seq)
    : pool_(pool), max_slots_(max_slots), max_blocks_(max_blocks_per_seq) {
  if (max_slots < 1 || max_blocks_per_seq < 1) throw std::invalid_argument("BlockTable: bad geometry");
  image_.assign(static_cast<size_t>(max_slots) * max_blocks_per_seq, 0);
  counts_.assign(max_slots, 0);
  dirty_.assign(max_slots, 0);
}

bool BlockTable::ensure_capacity(int slot, int64_t tokens) {
  if (slot < 0 || slot >= max_slots_) throw std::out_of_range("BlockTable: slot");
  const int need = pool_.blocks_for_tokens(tokens);
  if (need > max_blocks_) return false;
  const int have = counts_[slot];
  if (need <= have) return true;
  std::vector<int32_t> got;
  if (!pool_.allocate(need - have, got)) return false;
  int32_t* r = image_.data() + static_cast<size_t>(slot) * max_blocks_;
  for (int i = 0; i < need - have; ++i) r[have + i] = got[i];
  counts_[slot] = need;
  dirty_[slot] = 1;
  return true;
}

bool BlockTable::share_prefix(int dst, int src, int n_blocks) {
  if (dst < 0 || dst >= max_slots_ || src < 0 || src >= max_slots_) throw std::out_of_range("BlockTable: slot");
  if (counts_[dst] != 0 || n_blocks > counts_[src] || n_blocks > max_blocks_) return false;
  for (int i = 0; i < n_blocks; ++i) {
    const int32_t b = block_at(src, i);
    pool_.retain(b);
    image_[static_cast<size_t>(dst) * max_blocks_ + i] = b;
  }
  counts_[dst] = n_blocks;
  dirty_[dst] = 1;
  return true;
}

bool BlockTable::adopt(int dst, const int32_t* blocks, int n_blocks) {
  if (dst < 0 || dst >= max_slots_) throw std::out_of_range("BlockTable: slot");
  if (counts_[dst] != 0 || n_blocks < 0 || n_blocks > max_blocks_) return false;
  // all or nothing: a block that is not live (a stale cache entry, a foreign id) leaves the row and the pool untouched
  int held = 0;
  try {
    for (; held < n_blocks; ++held) pool_.retain(blocks[held]);
  } catch (const std::invalid_argument&) {
    for (int i = 0; i < held; ++i) pool_.release(blocks[i]);
    return false;
  }
  for (int i = 0; i < n_blocks; ++i) image_[static_cast<size_t>(dst) * max_blocks_ + i] = blocks[i];
  counts_[dst] = n_blocks;
  dirty_[dst] = 1;
  return true;
}

void BlockTable::free_slot(int slot) {
  if (slot < 0 || slot >= max_slots_) throw std::out_of_range("BlockTable: slot");
  int32_t* r = image_.data() + static_cast<size_t>(slot) * max_blocks_;
  for (int i = 0; i < counts_[slot]; ++i) {
    pool_.release(r[i]);
    r[i] = 0;
  }
  if (counts_[slot]) dirty_[slot] = 1;
  counts_[slot] = 0;
}

int64_t BlockTable::element_offset(int slot, int64_t pos) const {
  const int bt = pool_.block_tokens();
  const int64_t blk = pos / bt;
  if (slot < 0 || slot >= max_slots_ || blk >= counts_[slot]) throw std::out_of_range("BlockTable: position not mapped");
  return static_cast<int64_t>(block_at(slot, static_cast<int>(blk))) * bt + pos % bt;
}

std::vector<int> BlockTable::take_dirty_rows() {
  std::vector<int> rows;
  for (int s = 0; s < max_slots_; ++s)
    if (dirty_[s]) { rows.push_back(s); dirty_[s] = 0; }
  return rows;
}

}  // namespace pocket
