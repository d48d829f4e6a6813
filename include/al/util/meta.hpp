/**
 * @file meta.hpp
 * constexpr integer helpers used by the queues and allocators.
 * Parity: include/aluminum/utils/meta.hpp:38-110 (is_pow2, next_highest_pow2,
 * floor_log2, ceil_log2, num_pow2s_between, pow2_ar).
 */
#pragma once
#include <array>
#include <cstddef>
#include <cstdint>

namespace Al {
namespace internal {

constexpr bool is_pow2(uint64_t x) { return x != 0 && (x & (x - 1)) == 0; }

constexpr unsigned floor_log2(uint64_t x) {
  unsigned r = 0;
  while (x >>= 1) ++r;
  return r;
}

constexpr unsigned ceil_log2(uint64_t x) {
  return x <= 1 ? 0 : floor_log2(x - 1) + 1;
}

constexpr uint64_t next_highest_pow2(uint64_t x) {
  return x <= 1 ? 1 : (uint64_t{1} << ceil_log2(x));
}

/** Number of powers of two in the closed interval [lo, hi]. */
constexpr unsigned num_pow2s_between(uint64_t lo, uint64_t hi) {
  if (hi < lo || hi == 0) return 0;
  unsigned first = ceil_log2(lo == 0 ? 1 : lo);
  unsigned last = floor_log2(hi);
  return last >= first ? last - first + 1 : 0;
}

/** Array of the N consecutive powers of two starting at `start` (a power of two). */
template <size_t N>
constexpr std::array<uint64_t, N> pow2_ar(uint64_t start) {
  std::array<uint64_t, N> a{};
  uint64_t v = start;
  for (size_t i = 0; i < N; ++i) { a[i] = v; v <<= 1; }
  return a;
}

constexpr uint64_t round_up(uint64_t x, uint64_t m) { return (x + m - 1) / m * m; }
constexpr uint64_t ceil_div(uint64_t x, uint64_t m) { return (x + m - 1) / m; }

}  // namespace internal
}  // namespace Al
