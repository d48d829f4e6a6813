/**
 * @file mpsc_queue.hpp
 * Bounded lock-free multi-producer / single-consumer ring.
 *
 * Parity: include/aluminum/utils/mpsc_queue.hpp:43-185 (the input queue the
 * progress engine uses when several user threads enqueue concurrently).
 * Design: every cell carries a ticket; a producer claims a position with one
 * fetch-free CAS on the tail and publishes by advancing the cell's ticket, the
 * consumer frees the cell by advancing it by the ring size.  A cell that has
 * been claimed but not yet published simply makes the consumer see "empty",
 * so elements are delivered in claim order.
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
class MPSCQueue {
  struct alignas(AL_CACHE_LINE_SIZE) Cell {
    std::atomic<size_t> ticket;
    T value;
  };

 public:
  explicit MPSCQueue(size_t capacity)
      : cap_(next_highest_pow2(capacity)), mask_(cap_ - 1), cells_(new Cell[cap_]) {
    for (size_t i = 0; i < cap_; ++i) cells_[i].ticket.store(i, std::memory_order_relaxed);
  }
  MPSCQueue(const MPSCQueue&) = delete;
  MPSCQueue& operator=(const MPSCQueue&) = delete;

  bool try_push(const T& v) {
    size_t pos = tail_.load(std::memory_order_relaxed);
    for (;;) {
      Cell& c = cells_[pos & mask_];
      const size_t tk = c.ticket.load(std::memory_order_acquire);
      const intptr_t diff = static_cast<intptr_t>(tk) - static_cast<intptr_t>(pos);
      if (diff == 0) {
        if (tail_.compare_exchange_weak(pos, pos + 1, std::memory_order_relaxed)) {
          c.value = v;
          c.ticket.store(pos + 1, std::memory_order_release);
          return true;
        }
      } else if (diff < 0) {
        return false;  // full
      } else {
        pos = tail_.load(std::memory_order_relaxed);
      }
    }
  }
  void push(const T& v) {
    if (!try_push(v)) throw_al_exception("MPSC queue full");
  }
  bool peek(T& out) {
    Cell& c = cells_[head_ & mask_];
    if (c.ticket.load(std::memory_order_acquire) != head_ + 1) return false;
    out = c.value;
    return true;
  }
  void pop_always() {
    Cell& c = cells_[head_ & mask_];
    c.ticket.store(head_ + cap_, std::memory_order_release);
    ++head_;
  }
  bool pop(T& out) {
    if (!peek(out)) return false;
    pop_always();
    return true;
  }
  size_t capacity() const { return cap_; }

 private:
  const size_t cap_, mask_;
  std::unique_ptr<Cell[]> cells_;
  alignas(AL_DESTRUCTIVE_INTERFERENCE_SIZE) std::atomic<size_t> tail_{0};
  alignas(AL_DESTRUCTIVE_INTERFERENCE_SIZE) size_t head_ = 0;  // consumer-private
};

}  // namespace internal
}  // namespace Al
