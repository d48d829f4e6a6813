/**
 * @file debug.hpp
 * Argument checks run at every API entry when AL_DEBUG=1 (or
 * Al::tuning().debug_checks) - null buffers with non-zero counts, ranks out of
 * range, count vectors of the wrong length, mismatched MultiSendRecv lists,
 * overlapping send / receive ranges.
 * Parity: include/aluminum/debug_helpers.hpp:56-283 (compile-time gated there,
 * run-time gated here so one build serves both uses).
 */
#pragma once
#include <numeric>
#include <vector>

#include "al/base.hpp"
#include "al/tuning.hpp"

namespace Al {
namespace debug {

inline bool on() { return tuning().debug_checks; }

template <typename T>
void check_buffer(const T* buf, size_t count) {
  if (!on()) return;
  if (count > 0 && buf == nullptr) throw_al_exception("null buffer with non-zero count");
}
template <typename T>
void check_buffer_root(const T* buf, size_t count, int rank, int root) {
  if (rank == root) check_buffer(buf, count);
}
template <typename T>
void check_buffer_nonroot(const T* buf, size_t count, int rank, int root) {
  if (rank != root) check_buffer(buf, count);
}
template <typename T>
void check_overlap(const T* a, size_t na, const T* b, size_t nb) {
  if (!on() || !a || !b || internal::is_in_place(a)) return;
  if (a < b + nb && b < a + na) throw_al_exception("send and receive buffers overlap");
}
inline void check_rank(int rank, int size) {
  if (!on()) return;
  if (rank < 0 || rank >= size) throw_al_exception("rank ", rank, " out of range for a communicator of ", size);
}
inline void check_vector_is_comm_sized(const std::vector<size_t>& v, int size) {
  if (!on()) return;
  if ((int)v.size() != size) throw_al_exception("vector has ", v.size(), " entries, communicator has ", size, " ranks");
}
inline size_t get_rank_entry(const std::vector<size_t>& v, int rank) { return v.at((size_t)rank); }
inline size_t sum(const std::vector<size_t>& v) { return std::accumulate(v.begin(), v.end(), size_t{0}); }
inline void check_multisendrecv(size_t ns_buf, size_t ns_cnt, size_t ns_dst, size_t nr_buf, size_t nr_cnt, size_t nr_src) {
  if (ns_buf != ns_cnt || ns_buf != ns_dst) throw_al_exception("MultiSendRecv: send lists differ in length");
  if (nr_buf != nr_cnt || nr_buf != nr_src) throw_al_exception("MultiSendRecv: receive lists differ in length");
}
inline void check_inplace_multisendrecv(size_t n_buf, size_t n_cnt, size_t n_dst, size_t n_src) {
  if (n_buf != n_cnt || n_buf != n_dst || n_buf != n_src) throw_al_exception("in-place MultiSendRecv: lists differ in length");
}

}  // namespace debug
}  // namespace Al
