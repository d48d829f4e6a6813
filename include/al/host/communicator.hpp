/**
 * @file communicator.hpp
 * Communicator and type-erased operations of the host (CPU) backend.
 *
 * Role: what the reference's MPI backend provides - collectives and
 * point-to-point on host memory, blocking and non-blocking through the
 * progress engine (include/aluminum/mpi_impl.hpp, the headers under include/aluminum/mpi,
 * communicator at include/aluminum/mpi/communicator.hpp:49-97).  There is no
 * MPI underneath.  When all members are on one node they share a POSIX
 * shared-memory workspace per communicator and run the same flag protocol the
 * device kernels use (publish into own staging half -> post epoch flag to
 * every peer -> wait for every peer's flag -> pull / reduce), so the CPU ranks
 * double as a model of the device protocol that can be tested without a GPU.
 * When the members are on several nodes the communicator owns TCP connections
 * between all pairs and runs the operations as rounds of non-blocking
 * messages (src/host_net.cpp).
 */
#pragma once
#include <atomic>
#include <memory>
#include <string>
#include <vector>

#include "al/base.hpp"
#include "al/bootstrap.hpp"

namespace Al {
namespace internal {
namespace host {

/** Completion record shared by an operation and the request handed to the user. */
struct ReqState {
  std::atomic<int> status{0};  ///< 0 pending, 1 done, 2 failed
  std::string error;           ///< valid once status == 2
};
using Request = std::shared_ptr<ReqState>;

class Workspace;  // shared-memory segment + layout

enum class Coll {
  allreduce, reduce, reduce_scatter, allgather, alltoall, bcast, gather, scatter, barrier
};

/** One collective call with in-place conventions already resolved. */
struct CollArgs {
  Coll kind = Coll::barrier;
  const void* send = nullptr;   ///< nullptr: this rank contributes nothing
  void* recv = nullptr;         ///< nullptr: this rank receives nothing
  DType dt = DType::u8;
  ReductionOperator op = ReductionOperator::sum;
  int root = 0;
  size_t count = 0;             ///< uniform count (meaning depends on the op)
  bool vector = false;          ///< use the count/displacement vectors below
  std::vector<size_t> send_counts, send_displs, recv_counts, recv_displs;
};

/** One transfer of a point-to-point operation. */
struct P2PItem {
  bool is_send = false;
  int peer = -1;
  const void* sbuf = nullptr;
  void* rbuf = nullptr;
  size_t bytes = 0;
};

/** Counters of one communicator (this rank's view). */
struct CommStats {
  uint64_t collectives = 0;  ///< collective calls accepted
  uint64_t p2p_ops = 0;      ///< point-to-point calls accepted (a MultiSendRecv counts once)
  uint64_t bytes = 0;        ///< payload bytes this rank contributed or sent
  uint64_t failures = 0;     ///< operations that ended in an error (time-outs included)
};

}  // namespace host
}  // namespace internal

/**
 * Host communicator.  Move-only, like every communicator of the reference;
 * `copy()` makes a new communicator over the same ranks.  The "stream" of a
 * host communicator is a dummy int, kept for interface parity
 * (include/aluminum/mpi/communicator.hpp:49-60).
 */
class HostCommunicator {
 public:
  /** World communicator (collective over all ranks). */
  HostCommunicator();
  /** Communicator over a subset (collective over the members). */
  explicit HostCommunicator(const internal::Group& group);
  ~HostCommunicator();
  HostCommunicator(HostCommunicator&&) noexcept;
  HostCommunicator& operator=(HostCommunicator&&) noexcept;
  HostCommunicator(const HostCommunicator&) = delete;
  HostCommunicator& operator=(const HostCommunicator&) = delete;

  HostCommunicator copy(int /*stream*/ = 0) const { return HostCommunicator(group_); }
  /** Communicator over the listed world ranks, in that order; collective over those ranks only. */
  static HostCommunicator from_ranks(const std::vector<int>& world_ranks);
  /** MPI_Comm_split analogue. */
  HostCommunicator split(int color, int key) const { return HostCommunicator(group_.split(color, key)); }

  int rank() const { return group_.rank(); }
  int size() const { return group_.size(); }
  /** Rank among, and number of, the members that run on this rank's node (the reference's node-local communicator, mpi_comm_and_stream_wrapper.hpp:46-129). */
  int local_rank() const;
  int local_size() const;
  /** Collective: the communicator of the members on this rank's node, ordered as here (role of get_local_comm()). */
  HostCommunicator local() const;
  int get_stream() const { return 0; }
  const internal::Group& group() const { return group_; }

  /** Start a collective; returns when done if `req` is null, else hands back a request. */
  void collective(internal::host::CollArgs&& args, internal::host::Request* req);
  /** Start a set of sends/receives that progress together. */
  void p2p(std::vector<internal::host::P2PItem>&& items, internal::host::Request* req, const char* name);

  /** Counters since creation. */
  internal::host::CommStats stats() const;
  /**
   * Put the communicator into the failed state on this rank: operations in
   * flight end with an error at their next progress step and later calls
   * throw.  The reference has no recovery path; the documented one here is
   * abort() on every surviving rank followed by a new communicator.
   */
  void abort(const std::string& why = "aborted by the caller");
  bool failed() const;

  struct Impl;
  Impl* impl() const { return impl_.get(); }

 private:
  internal::Group group_;
  std::unique_ptr<Impl> impl_;
};

}  // namespace Al
