/**
 * @file resolve.hpp
 * Turns one API call (operation, buffers, counts, in-place flag, root) into a
 * backend-neutral description with the in-place buffer conventions already
 * applied.  Both the host and the device backend consume it, so the
 * conventions live in exactly one place.
 *
 * Conventions (docs/comm.rst of the reference; include/aluminum/nccl_impl.hpp:
 * 1105-1111,1190-1205,1224-1234,1340-1343; include/aluminum/mpi/reduce.hpp:39-49,
 * mpi/scatter.hpp:39-51):
 *   reduce_scatter  in place: buffer holds count*p inputs, result in its first `count`
 *   allgather       in place: own slice already sits at rank*count
 *   gather          in place: root's slice sits at root*count of its buffer; a
 *                   non-root's buffer is its slice
 *   scatter         in place: root's buffer is the whole send vector and its
 *                   own slice stays where it is; a non-root's buffer receives
 */
#pragma once
#include <vector>

#include "al/base.hpp"

namespace Al {
namespace internal {

enum class OpKind {
  allreduce, reduce, reduce_scatter, allgather, alltoall, bcast, gather, scatter, barrier
};

struct Resolved {
  OpKind kind = OpKind::barrier;
  const void* send = nullptr;
  void* recv = nullptr;
  size_t count = 0;
  bool vector = false;
  std::vector<size_t> send_counts, send_displs, recv_counts, recv_displs;
  int root = 0;
  ReductionOperator op = ReductionOperator::sum;
  DType dt = DType::u8;
  bool in_place = false;  ///< the call used the single-buffer form: send and recv alias on purpose
};

/** Elements of the (resolved) send and receive buffers that the operation reads / writes on `rank`. */
struct Extent { size_t send_elems = 0, recv_elems = 0; };
inline Extent extent_of(const Resolved& r, int rank, int size) {
  Extent e;
  const size_t p = (size_t)size;
  auto span = [&](const std::vector<size_t>& c, const std::vector<size_t>& d) {
    size_t m = 0;
    for (size_t i = 0; i < c.size(); ++i) m = m > (d.empty() ? 0 : d[i]) + c[i] ? m : (d.empty() ? 0 : d[i]) + c[i];
    return m;
  };
  switch (r.kind) {
    case OpKind::allreduce: case OpKind::reduce: e.send_elems = e.recv_elems = r.count; break;
    case OpKind::bcast: e.send_elems = rank == r.root ? r.count : 0; e.recv_elems = rank == r.root ? 0 : r.count; break;
    case OpKind::reduce_scatter:
      if (r.vector) { e.send_elems = span(r.send_counts, r.send_displs); e.recv_elems = r.recv_counts[(size_t)rank]; }
      else { e.send_elems = r.count * p; e.recv_elems = r.count; }
      break;
    case OpKind::allgather:
      if (r.vector) { e.send_elems = r.send_counts[(size_t)rank]; e.recv_elems = span(r.recv_counts, r.recv_displs); }
      else { e.send_elems = r.count; e.recv_elems = r.count * p; }
      break;
    case OpKind::alltoall:
      if (r.vector) { e.send_elems = span(r.send_counts, r.send_displs); e.recv_elems = span(r.recv_counts, r.recv_displs); }
      else { e.send_elems = e.recv_elems = r.count * p; }
      break;
    case OpKind::gather:
      if (r.vector) { e.send_elems = r.send_counts[(size_t)rank]; e.recv_elems = span(r.recv_counts, r.recv_displs); }
      else { e.send_elems = r.count; e.recv_elems = r.count * p; }
      break;
    case OpKind::scatter:
      if (r.vector) { e.send_elems = span(r.send_counts, r.send_displs); e.recv_elems = r.recv_counts[(size_t)rank]; }
      else { e.send_elems = r.count * p; e.recv_elems = r.count; }
      break;
    case OpKind::barrier: break;
  }
  if (!r.send) e.send_elems = 0;
  if (!r.recv) e.recv_elems = 0;
  return e;
}

inline const char* op_kind_name(OpKind k) {
  static const char* n[] = {"allreduce", "reduce", "reduce_scatter", "allgather", "alltoall",
                            "bcast", "gather", "scatter", "barrier"};
  return n[(int)k];
}

inline const void* offset_ptr(const void* p, size_t elems, DType dt) {
  return (const char*)p + elems * dtype_size(dt);
}

/** Uniform-count collectives. `send == IN_PLACE` selects the in-place form on `recv`. */
inline Resolved resolve_uniform(OpKind kind, DType dt, const void* send, void* recv, size_t count,
                                ReductionOperator op, int root, int rank, int /*size*/) {
  Resolved r;
  r.kind = kind; r.dt = dt; r.count = count; r.op = op; r.root = root;
  const bool ip = is_in_place(send);
  r.in_place = ip || kind == OpKind::bcast;
  switch (kind) {
    case OpKind::allreduce: case OpKind::reduce: case OpKind::reduce_scatter: case OpKind::alltoall:
      r.send = ip ? recv : send; r.recv = recv; break;
    case OpKind::allgather:
      r.send = ip ? offset_ptr(recv, (size_t)rank * count, dt) : send; r.recv = recv; break;
    case OpKind::bcast:
      r.send = recv; r.recv = recv; break;
    case OpKind::gather:
      if (rank == root) { r.send = ip ? offset_ptr(recv, (size_t)root * count, dt) : send; r.recv = recv; }
      else { r.send = ip ? recv : send; r.recv = nullptr; }
      break;
    case OpKind::scatter:
      if (rank == root) { r.send = ip ? recv : send; r.recv = ip ? nullptr : recv; }
      else { r.send = nullptr; r.recv = recv; }
      break;
    case OpKind::barrier: break;
  }
  if (kind == OpKind::reduce && rank != root) r.recv = nullptr;
  return r;
}

inline std::vector<size_t> prefix_displs(const std::vector<size_t>& counts) {
  std::vector<size_t> d(counts.size());
  size_t run = 0;
  for (size_t i = 0; i < counts.size(); ++i) { d[i] = run; run += counts[i]; }
  return d;
}

/** Vector collectives. Unused tables may be left empty by the caller. */
inline Resolved resolve_vector(OpKind kind, DType dt, const void* send, void* recv,
                               std::vector<size_t> send_counts, std::vector<size_t> send_displs,
                               std::vector<size_t> recv_counts, std::vector<size_t> recv_displs,
                               ReductionOperator op, int root, int rank, int size) {
  Resolved r;
  r.kind = kind; r.dt = dt; r.op = op; r.root = root; r.vector = true;
  const bool ip = is_in_place(send);
  r.in_place = ip;
  const size_t p = (size_t)size;
  switch (kind) {
    case OpKind::reduce_scatter:  // counts = per-rank output lengths, inputs contiguous in rank order
      if (recv_counts.size() != p) throw_al_exception("reduce_scatterv: counts must have one entry per rank");
      r.recv_counts = recv_counts; r.send_counts = recv_counts; r.send_displs = prefix_displs(recv_counts);
      r.recv_displs.assign(p, 0);
      r.send = ip ? recv : send; r.recv = recv; break;
    case OpKind::allgather:
      if (recv_counts.size() != p || recv_displs.size() != p) throw_al_exception("allgatherv: counts/displs must have one entry per rank");
      r.recv_counts = recv_counts; r.recv_displs = recv_displs;
      r.send_counts = recv_counts; r.send_displs.assign(p, 0);
      r.send = ip ? offset_ptr(recv, recv_displs[(size_t)rank], dt) : send; r.recv = recv; break;
    case OpKind::alltoall:
      if (ip) { send_counts = recv_counts; send_displs = recv_displs; }
      if (send_counts.size() != p || send_displs.size() != p || recv_counts.size() != p || recv_displs.size() != p)
        throw_al_exception("alltoallv: counts/displs must have one entry per rank");
      r.send_counts = send_counts; r.send_displs = send_displs; r.recv_counts = recv_counts; r.recv_displs = recv_displs;
      r.send = ip ? recv : send; r.recv = recv; break;
    case OpKind::gather:  // counts/displs describe the root's receive layout
      if (recv_counts.size() != p || recv_displs.size() != p) throw_al_exception("gatherv: counts/displs must have one entry per rank");
      r.recv_counts = recv_counts; r.recv_displs = recv_displs; r.send_counts = recv_counts; r.send_displs.assign(p, 0);
      if (rank == root) { r.send = ip ? offset_ptr(recv, recv_displs[(size_t)root], dt) : send; r.recv = recv; }
      else { r.send = ip ? recv : send; r.recv = nullptr; }
      break;
    case OpKind::scatter:  // counts/displs describe the root's send layout
      if (send_counts.size() != p || send_displs.size() != p) throw_al_exception("scatterv: counts/displs must have one entry per rank");
      r.send_counts = send_counts; r.send_displs = send_displs; r.recv_counts = send_counts; r.recv_displs.assign(p, 0);
      if (rank == root) { r.send = ip ? recv : send; r.recv = ip ? nullptr : recv; }
      else { r.send = nullptr; r.recv = recv; }
      break;
    default: throw_al_exception("no vector form of ", op_kind_name(kind));
  }
  return r;
}

}  // namespace internal
}  // namespace Al
