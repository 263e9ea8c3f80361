#include "block_pool.hpp"

#include <stdexcept>

namespace pocket {

BlockPool::BlockPool(int num_blocks, int block_tokens) : num_blocks_(num_blocks), block_tokens_(block_tokens) {
  if (num_blocks < 2 || block_tokens < 1) throw std::invalid_argument("BlockPool: need >= 2 blocks and a positive block size");
  refs_.assign(num_blocks, 0);
  free_.reserve(num_blocks - 1);
  for (int b = num_blocks - 1; b >= 1; --b) free_.push_back(b);   // pop_back hands out 1, 2, 3, ...
}

int BlockPool::free_blocks() const {
  std::lock_guard<std::mutex> g(mu_);
  return static_cast<int>(free_.size());
}

bool BlockPool::allocate(int n, std::vector<int32_t>& out) {
  if (n < 0) throw std::invalid_argument("BlockPool::allocate: negative count");
  std::lock_guard<std::mutex> g(mu_);
  if (static_cast<size_t>(n) > free_.size()) return false;
  for (int i = 0; i < n; ++i) {
    int32_t b = free_.back();
    free_.pop_back();
    refs_[b] = 1;
    out.push_back(b);
  }
  return true;
}

void BlockPool::retain(int32_t block) {
  std::lock_guard<std::mutex> g(mu_);
  if (block < 1 || block >= num_blocks_ || refs_[block] <= 0) throw std::invalid_argument("BlockPool::retain: block not live");
  ++refs_[block];
}

void BlockPool::release(int32_t block) {
  std::lock_guard<std::mutex> g(mu_);
  if (block < 1 || block >= num_blocks_ || refs_[block] <= 0) throw std::invalid_argument("BlockPool::release: block not live");
  if (--refs_[block] == 0) free_.push_back(block);
}

void BlockPool::release_all(const std::vector<int32_t>& blocks) {
  for (int32_t b : blocks) release(b);
}

int BlockPool::refcount(int32_t block) const {
  std::lock_guard<std::mutex> g(mu_);
  return (block >= 0 && block < num_blocks_) ? refs_[block] : 0;
}

}  // namespace pocket
