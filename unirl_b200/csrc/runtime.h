#pragma once
#include <stdint.h>
#include <vector>

namespace ub {

class BlockAllocator {
 public:
  explicit BlockAllocator(int64_t num_pages);
  void reset();
  std::vector<int64_t> allocate(int64_t n);
  void free(const std::vector<int64_t>& pages);
  int64_t num_free() const { return static_cast<int64_t>(free_.size()); }
  int64_t num_pages() const { return num_pages_; }

 private:
  int64_t num_pages_;
  std::vector<int64_t> free_;
};

}  // namespace ub
