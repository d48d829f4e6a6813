/**
 * @file spsc_queue.hpp
 * Bounded wait-free single-producer / single-consumer ring of values.
 *
 * Parity: include/aluminum/utils/spsc_queue.hpp:46-141 (push / pop /
 * pop_always / peek on a power-of-two ring with cache-line-separated
 * indices).  This version additionally keeps, on each side, a private copy of
 * the other side's index so that the common case touches no shared line, and
 * reports overflow through the return value instead of aborting.
 */
#pragma once
#include <atomic>
#include <cstddef>
#include <memory>

#include "al/base.hpp"
#include "al/util/meta.hpp"

namespace Al {
namespace internal {

template <typename T>
class SPSCQueue {
 public:
  explicit SPSCQueue(size_t capacity)
      : cap_(next_highest_pow2(capacity)), mask_(cap_ - 1), ring_(new T[cap_]) {
    if (capacity == 0) throw_al_exception("SPSCQueue capacity must be positive");
  }
  SPSCQueue(const SPSCQueue&) = delete;
  SPSCQueue& operator=(const SPSCQueue&) = delete;

  /** Producer: false when the ring is full. */
  bool try_push(const T& v) {
    const size_t t = tail_.load(std::memory_order_relaxed);
    if (t - head_seen_ >= cap_) {
      head_seen_ = head_.load(std::memory_order_acquire);
      if (t - head_seen_ >= cap_) return false;
    }
    ring_[t & mask_] = v;
    tail_.store(t + 1, std::memory_order_release);
    return true;
  }
  /** Producer: throws when the ring is full. */
  void push(const T& v) {
    if (!try_push(v)) throw_al_exception("SPSC queue full");
  }
  /** Consumer: false when empty. */
  bool pop(T& out) {
    const size_t h = head_.load(std::memory_order_relaxed);
    if (h == tail_seen_) {
      tail_seen_ = tail_.load(std::memory_order_acquire);
      if (h == tail_seen_) return false;
    }
    out = ring_[h & mask_];
    head_.store(h + 1, std::memory_order_release);
    return true;
  }
  /** Consumer: look at the front element without removing it. */
  bool peek(T& out) {
    const size_t h = head_.load(std::memory_order_relaxed);
    if (h == tail_seen_) {
      tail_seen_ = tail_.load(std::memory_order_acquire);
      if (h == tail_seen_) return false;
    }
    out = ring_[h & mask_];
    return true;
  }
  /** Consumer: drop the front element; only valid after a successful peek(). */
  void pop_always() {
    head_.store(head_.load(std::memory_order_relaxed) + 1, std::memory_order_release);
  }
  size_t size_approx() const {
    return tail_.load(std::memory_order_acquire) - head_.load(std::memory_order_acquire);
  }
  size_t capacity() const { return cap_; }

 private:
  const size_t cap_, mask_;
  std::unique_ptr<T[]> ring_;
  alignas(AL_DESTRUCTIVE_INTERFERENCE_SIZE) std::atomic<size_t> head_{0};
  size_t tail_seen_ = 0;  // consumer-private
  alignas(AL_DESTRUCTIVE_INTERFERENCE_SIZE) std::atomic<size_t> tail_{0};
  size_t head_seen_ = 0;  // producer-private
};

}  // namespace internal
}  // namespace Al
