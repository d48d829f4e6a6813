/**
 * @file caching_allocator.hpp
 * Thread-safe size-class caching allocator for host, pinned-host and device
 * memory.
 *
 * Parity: include/aluminum/utils/caching_allocator.hpp:47-246 (size-binned
 * free lists, bins computed constexpr, allocations above the largest bin are
 * never cached) and the MemoryType enum at :98-107.
 *
 * Design: bins are "quarter octaves" - for every power of two 2^k the classes
 * 2^k, 1.25*2^k, 1.5*2^k, 1.75*2^k - so the class index follows from two bit
 * operations with no table search, and internal waste is bounded by 25 %.
 */
#pragma once
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "al/base.hpp"
#include "al/util/meta.hpp"

namespace Al {

enum class MemoryType { HOST, CUDA_PINNED_HOST, CUDA };

namespace internal {

struct SizeClasses {
  static constexpr unsigned min_log2 = 6;    // 64 B
  static constexpr unsigned max_log2 = 28;   // 256 MiB
  static constexpr unsigned steps = 4;
  static constexpr size_t num_bins = (max_log2 - min_log2) * steps + 1;

  /** Smallest class index whose size is >= bytes; num_bins if above the largest class. */
  static constexpr size_t bin_of(size_t bytes) {
    if (bytes <= (size_t{1} << min_log2)) return 0;
    if (bytes > (size_t{1} << max_log2)) return num_bins;
    const unsigned k = floor_log2(bytes);             // 2^k <= bytes
    const size_t base = size_t{1} << k;
    if (bytes == base) return (k - min_log2) * steps;
    const size_t quarter = base >> 2;
    const size_t step = (bytes - base + quarter - 1) / quarter;  // 1..4
    return (k - min_log2) * steps + step;
  }
  static constexpr size_t bin_size(size_t bin) {
    const unsigned k = min_log2 + static_cast<unsigned>(bin / steps);
    const size_t base = size_t{1} << k;
    return base + (base >> 2) * (bin % steps);
  }
};

static_assert(SizeClasses::bin_of(64) == 0, "bin math");
static_assert(SizeClasses::bin_size(SizeClasses::bin_of(65)) == 80, "bin math");
static_assert(SizeClasses::bin_size(SizeClasses::bin_of(1000)) == 1024, "bin math");
static_assert(SizeClasses::bin_size(SizeClasses::bin_of(1025)) == 1280, "bin math");
static_assert(SizeClasses::bin_of((size_t{1} << 28) + 1) == SizeClasses::num_bins, "bin math");

/**
 * @tparam RawAlloc has `void* allocate(size_t bytes)` and
 *                  `void deallocate(void*, size_t bytes)`.
 */
template <typename RawAlloc>
class CachingAllocator {
 public:
  CachingAllocator() = default;
  explicit CachingAllocator(RawAlloc raw) : raw_(std::move(raw)) {}
  ~CachingAllocator() { /* clear() must be called while the backing runtime is alive */ }

  void* allocate(size_t bytes) {
    if (bytes == 0) bytes = 1;
    const size_t bin = SizeClasses::bin_of(bytes);
    size_t actual = bytes;
    void* p = nullptr;
    if (bin < SizeClasses::num_bins) {
      actual = SizeClasses::bin_size(bin);
      std::lock_guard<std::mutex> g(mu_);
      auto& fl = free_[bin];
      if (!fl.empty()) {
        p = fl.back();
        fl.pop_back();
        ++hits_;
      }
    }
    if (!p) {
      p = raw_.allocate(actual);
      ++misses_;
    }
    std::lock_guard<std::mutex> g(mu_);
    live_[p] = bin;
    live_bytes_[p] = actual;
    return p;
  }

  void release(void* p) {
    if (!p) return;
    size_t bin, actual;
    {
      std::lock_guard<std::mutex> g(mu_);
      auto it = live_.find(p);
      if (it == live_.end()) throw_al_exception("release of a pointer this pool did not allocate");
      bin = it->second;
      actual = live_bytes_[p];
      live_.erase(it);
      live_bytes_.erase(p);
      if (bin < SizeClasses::num_bins) {
        free_[bin].push_back(p);
        return;
      }
    }
    raw_.deallocate(p, actual);
  }

  /** Return every cached (idle) block to the system. */
  void clear() {
    std::lock_guard<std::mutex> g(mu_);
    for (size_t b = 0; b < SizeClasses::num_bins; ++b) {
      for (void* p : free_[b]) raw_.deallocate(p, SizeClasses::bin_size(b));
      free_[b].clear();
    }
  }
  size_t hits() const { return hits_; }
  size_t misses() const { return misses_; }
  size_t live_blocks() {
    std::lock_guard<std::mutex> g(mu_);
    return live_.size();
  }

 private:
  RawAlloc raw_;
  std::mutex mu_;
  std::vector<void*> free_[SizeClasses::num_bins];
  std::unordered_map<void*, size_t> live_;
  std::unordered_map<void*, size_t> live_bytes_;
  size_t hits_ = 0, misses_ = 0;
};

}  // namespace internal
}  // namespace Al
