// Host-side runtime pieces that sit on the decode critical path between kernel launches.
//
// BlockAllocator: LIFO free-list over KV-cache page ids with O(1) allocate/free and bulk reservation,
// the native counterpart of the Python allocator in rollout/engine/native_ar/kv_cache.py.
#include "runtime.h"

#include <stdexcept>
#include <string>

namespace ub {

BlockAllocator::BlockAllocator(int64_t num_pages) : num_pages_(num_pages) { reset(); }

void BlockAllocator::reset() {
  free_.resize(static_cast<size_t>(num_pages_));
  for (int64_t i = 0; i < num_pages_; ++i) free_[static_cast<size_t>(i)] = num_pages_ - 1 - i;
}

std::vector<int64_t> BlockAllocator::allocate(int64_t n) {
  if (n < 0 || static_cast<size_t>(n) > free_.size())
    throw std::runtime_error("KV cache exhausted: need " + std::to_string(n) + " pages, " + std::to_string(free_.size()) + " free of " +
                             std::to_string(num_pages_));
  std::vector<int64_t> out(static_cast<size_t>(n));
  for (int64_t i = 0; i < n; ++i) {
    out[static_cast<size_t>(i)] = free_.back();
    free_.pop_back();
  }
  return out;
}

void BlockAllocator::free(const std::vector<int64_t>& pages) {
  for (auto it = pages.rbegin(); it != pages.rend(); ++it) free_.push_back(*it);
}

}  // namespace ub
