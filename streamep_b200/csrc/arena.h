// Best-fit free-list allocator over one contiguous range of device addresses.
//
// Buffers that peers write into (pools, per-slot arrays, arrival counters, accumulators) must sit
// at addresses every rank has mapped, so they cannot come from torch's caching allocator.  The
// arena hands out sub-ranges of one peer-mapped slab; tensors created over them return their
// block when the last reference dies, which lets autograd keep a pool alive from forward to
// backward without any extra bookkeeping.
//
// Stream safety: a tensor's last reference can die while kernels that use its block are still
// queued.  release_deferred() parks the block behind a fence (the runtime records an event on every
// stream it has launched on); the block becomes reusable only once the fence reports completion.
// allocate() sweeps the parked blocks first and, when the arena is exhausted, waits for them.
//
// The reference allocates one IPC slab per rank and carves ring buffers out of it at fixed
// offsets (csrc/stream_ep.cpp:187-221, csrc/kernels/buffer.cuh:8-129); it allocates per-dispatch
// tensors with torch::empty because only its rings are written by peers.
#pragma once

#include <cstddef>
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <vector>

namespace sep {

// Completion of the work that may still touch a released block.
struct ArenaFence {
  virtual ~ArenaFence() = default;
  virtual bool ready() = 0;   // non-blocking
  virtual void wait() = 0;    // blocking
};

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
    parked_.clear();
    in_use_ = 0;
    high_water_ = 0;
    parked_bytes_ = 0;
  }

  // Returns the offset of a block of at least `bytes` bytes.
  size_t allocate(size_t bytes) {
    const size_t need = bytes == 0 ? kAlign : (bytes + kAlign - 1) / kAlign * kAlign;
    std::lock_guard<std::mutex> g(mu_);
    sweep_locked(false);
    auto find = [&] {
      auto best = free_.end();
      for (auto it = free_.begin(); it != free_.end(); ++it)
        if (it->second >= need && (best == free_.end() || it->second < best->second)) best = it;
      return best;
    };
    auto best = find();
    if (best == free_.end() && !parked_.empty()) {   // wait for blocks whose last users are still running
      sweep_locked(true);
      best = find();
    }
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

  // The block at `off` is no longer referenced, but work that uses it may still be queued: it becomes
  // reusable once `fence` is ready.  Counts as released for bytes_in_use().
  void release_deferred(size_t off, std::shared_ptr<ArenaFence> fence) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = used_.find(off);
    if (it == used_.end()) return;
    if (!fence || fence->ready()) { release_locked(off); return; }
    parked_bytes_ += it->second;
    parked_.push_back({off, std::move(fence)});
  }
  // Returns blocks whose fence completed to the free list (`block` = wait for every fence).
  void sweep(bool block = false) {
    std::lock_guard<std::mutex> g(mu_);
    sweep_locked(block);
  }
  size_t num_parked() const { return parked_.size(); }

  void release(size_t off) {
    std::lock_guard<std::mutex> g(mu_);
    release_locked(off);
  }

  size_t bytes_in_use() const { return in_use_ - parked_bytes_; }
  size_t high_water() const { return high_water_; }
  size_t capacity() const { return end_ - begin_; }
  size_t num_free_blocks() const { return free_.size(); }

 private:
  struct Parked { size_t off; std::shared_ptr<ArenaFence> fence; };

  void sweep_locked(bool block) {
    size_t kept = 0;
    for (size_t i = 0; i < parked_.size(); ++i) {
      Parked& pk = parked_[i];
      if (block) pk.fence->wait();
      if (block || pk.fence->ready()) {
        auto it = used_.find(pk.off);
        if (it != used_.end()) parked_bytes_ -= it->second;
        release_locked(pk.off);
      } else {
        if (kept != i) parked_[kept] = std::move(pk);
        ++kept;
      }
    }
    parked_.resize(kept);
  }

  void release_locked(size_t off) {
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

  std::mutex mu_;
  std::map<size_t, size_t> free_;   // offset -> size
  std::map<size_t, size_t> used_;
  std::vector<Parked> parked_;
  size_t begin_ = 0, end_ = 0, in_use_ = 0, high_water_ = 0, parked_bytes_ = 0;
};

}  // namespace sep
