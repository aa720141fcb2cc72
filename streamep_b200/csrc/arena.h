// Best-fit free-list allocator over one contiguous range of device addresses.
//
// Buffers that peers write into (pools, per-slot arrays, arrival counters, accumulators) must sit
// at addresses every rank has mapped, so they cannot come from torch's caching allocator.  The
// arena hands out sub-ranges of one peer-mapped slab; tensors created over them return their
// block when the last reference dies, which lets autograd keep a pool alive from forward to
// backward without any extra bookkeeping.
//
// The reference allocates one IPC slab per rank and carves ring buffers out of it at fixed
// offsets (csrc/stream_ep.cpp:187-221, csrc/kernels/buffer.cuh:8-129); it allocates per-dispatch
// tensors with torch::empty because only its rings are written by peers.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <mutex>
#include <stdexcept>
#include <string>

namespace sep {

class Arena {
 public:
  static constexpr size_t kAlign = 1024;

  Arena() = default;
  Arena(size_t offset, size_t size) { reset(offset, size); }

  void reset(size_t offset, size_t size) {
    std::lock_guard<std::mutex> g(mu_);
    free_.clear();
    used_.clear();
    begin_ = (offset + kAlign - 1) / kAlign * kAlign;
    end_ = offset + size;
    if (end_ > begin_) free_[begin_] = end_ - begin_;
    in_use_ = 0;
    high_water_ = 0;
  }

  // Returns the offset of a block of at least `bytes` bytes.
  size_t allocate(size_t bytes) {
    const size_t need = bytes == 0 ? kAlign : (bytes + kAlign - 1) / kAlign * kAlign;
    std::lock_guard<std::mutex> g(mu_);
    auto best = free_.end();
    for (auto it = free_.begin(); it != free_.end(); ++it)
      if (it->second >= need && (best == free_.end() || it->second < best->second)) best = it;
    if (best == free_.end())
      throw std::runtime_error("streamep_b200: symmetric arena exhausted (need " + std::to_string(need) +
                               " bytes, in use " + std::to_string(in_use_) + " of " +
                               std::to_string(end_ - begin_) + "); construct the Buffer with a larger num_nvl_bytes");
    const size_t off = best->first, sz = best->second;
    free_.erase(best);
    if (sz > need) free_[off + need] = sz - need;
    used_[off] = need;
    in_use_ += need;
    if (in_use_ > high_water_) high_water_ = in_use_;
    return off;
  }

  void release(size_t off) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = used_.find(off);
    if (it == used_.end()) return;
    size_t sz = it->second;
    used_.erase(it);
    in_use_ -= sz;
    auto next = free_.lower_bound(off);
    if (next != free_.end() && off + sz == next->first) {   // merge with the block after
      sz += next->second;
      next = free_.erase(next);
    }
    if (next != free_.begin()) {                            // merge with the block before
      auto prev = std::prev(next);
      if (prev->first + prev->second == off) {
        prev->second += sz;
        return;
      }
    }
    free_[off] = sz;
  }

  size_t bytes_in_use() const { return in_use_; }
  size_t high_water() const { return high_water_; }
  size_t capacity() const { return end_ - begin_; }
  size_t num_free_blocks() const { return free_.size(); }

 private:
  std::mutex mu_;
  std::map<size_t, size_t> free_;   // offset -> size
  std::map<size_t, size_t> used_;
  size_t begin_ = 0, end_ = 0, in_use_ = 0, high_water_ = 0;
};

}  // namespace sep
