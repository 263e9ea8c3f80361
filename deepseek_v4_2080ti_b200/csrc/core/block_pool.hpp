// Fixed-size KV block allocator: LIFO free list, per-block reference counts (prefix sharing),
// all-or-nothing multi-block allocation.  Block 0 is never handed out: decode batches park the
// K/V rows of padded lanes there.  (Role of cpp_engine/include/block_pool.hpp:24-68.)
#pragma once
#include <cstdint>
#include <mutex>
#include <vector>

namespace pocket {

class BlockPool {
 public:
  BlockPool(int num_blocks, int block_tokens);
  int block_tokens() const { return block_tokens_; }
  int total_blocks() const { return num_blocks_ - 1; }      // usable (block 0 reserved)
  int free_blocks() const;
  int blocks_for_tokens(int64_t tokens) const { return static_cast<int>((tokens + block_tokens_ - 1) / block_tokens_); }
  // Appends n block ids to out and returns true, or leaves everything untouched and returns false.
  bool allocate(int n, std::vector<int32_t>& out);
  void retain(int32_t block);                                // +1 reference (shared prefix)
  void release(int32_t block);                               // -1; returns to the free list at zero
  void release_all(const std::vector<int32_t>& blocks);
  int refcount(int32_t block) const;

 private:
  const int num_blocks_, block_tokens_;
  mutable std::mutex mu_;
  std::vector<int32_t> free_;
  std::vector<int32_t> refs_;
};

}  // namespace pocket
