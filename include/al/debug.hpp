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
#include "al/resolve.hpp"
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
/**
 * Checks of one resolved collective, whatever the operation: a buffer that the operation reads or
 * writes on this rank must not be null (on rooted operations only the significant side is looked
 * at: the root's receive buffer of a gather, a non-root's send buffer of a reduce, ...), and the
 * out-of-place forms must not be given overlapping send and receive ranges.
 */
inline void check_resolved(const internal::Resolved& r, bool send_given, bool recv_given, int rank, int size) {
  if (!on()) return;
  if (r.root < 0 || r.root >= size) throw_al_exception("root ", r.root, " out of range for a communicator of ", size);
  // what the operation needs on this rank, from the counts alone (extent_of answers 0 for a null pointer)
  internal::Resolved probe = r;
  probe.send = probe.send ? probe.send : (const void*)1;
  probe.recv = probe.recv ? probe.recv : (void*)1;
  const internal::Extent need = internal::extent_of(probe, rank, size);
  const bool reads = r.kind != internal::OpKind::barrier && !(r.kind == internal::OpKind::scatter && rank != r.root) &&
                     !(r.kind == internal::OpKind::bcast && rank != r.root);
  const bool writes = r.kind != internal::OpKind::barrier && !((r.kind == internal::OpKind::reduce || r.kind == internal::OpKind::gather) && rank != r.root) &&
                      !(r.kind == internal::OpKind::bcast && rank == r.root) &&
                      !(r.kind == internal::OpKind::scatter && rank == r.root && r.in_place);
  if (reads && need.send_elems > 0 && !send_given)
    throw_al_exception(internal::op_kind_name(r.kind), ": null send buffer with ", need.send_elems, " elements to send on rank ", rank);
  if (writes && need.recv_elems > 0 && !recv_given)
    throw_al_exception(internal::op_kind_name(r.kind), ": null receive buffer with ", need.recv_elems, " elements to receive on rank ", rank);
  if (!r.in_place && r.send && r.recv && need.send_elems && need.recv_elems) {
    const size_t esz = dtype_size(r.dt);
    const char* a = (const char*)r.send;
    const char* b = (const char*)r.recv;
    if (a < b + need.recv_elems * esz && b < a + need.send_elems * esz)
      throw_al_exception(internal::op_kind_name(r.kind), ": send and receive buffers overlap (use the in-place form)");
  }
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
