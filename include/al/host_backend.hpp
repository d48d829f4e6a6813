/**
 * @file host_backend.hpp
 * The CPU backend: collectives and point-to-point on host memory, through
 * shared memory between the ranks of one node and through sockets between
 * nodes, blocking or through the progress engine.
 *
 * Parity: Al::MPIBackend (include/aluminum/mpi_impl.hpp:112-990): same static
 * member names, `comm_type`, `req_type`, `null_req`, algorithm enums (all
 * aliases of `automatic`, as in mpi_impl.hpp:83-109) and Test/Wait semantics -
 * except that Test returns true on the call that observes completion (the
 * reference returns false once more, mpi_impl.hpp:967-976) and a failed
 * operation surfaces as an exception from Test/Wait.
 */
#pragma once
#include <thread>

#include "al/host/communicator.hpp"
#include "al/resolve.hpp"

namespace Al {

enum class HostAlgo { automatic };

class HostBackend {
 public:
  using comm_type = HostCommunicator;
  using req_type = internal::host::Request;
  static constexpr std::nullptr_t null_req = nullptr;
  using allreduce_algo_type = HostAlgo;  using reduce_algo_type = HostAlgo;
  using reduce_scatter_algo_type = HostAlgo;  using reduce_scatterv_algo_type = HostAlgo;
  using allgather_algo_type = HostAlgo;  using allgatherv_algo_type = HostAlgo;
  using alltoall_algo_type = HostAlgo;  using alltoallv_algo_type = HostAlgo;
  using barrier_algo_type = HostAlgo;  using bcast_algo_type = HostAlgo;
  using gather_algo_type = HostAlgo;  using gatherv_algo_type = HostAlgo;
  using scatter_algo_type = HostAlgo;  using scatterv_algo_type = HostAlgo;
  static std::string Name() { return "HostBackend"; }

  /** Run a resolved collective; `req == nullptr` blocks the caller. */
  static void run(internal::Resolved&& r, comm_type& comm, req_type* req, int /*algo*/ = 0) {
    internal::host::CollArgs a;
    a.kind = (internal::host::Coll)(int)r.kind;
    a.send = r.send; a.recv = r.recv; a.dt = r.dt; a.op = r.op; a.root = r.root; a.count = r.count;
    a.vector = r.vector;
    a.send_counts = std::move(r.send_counts); a.send_displs = std::move(r.send_displs);
    a.recv_counts = std::move(r.recv_counts); a.recv_displs = std::move(r.recv_displs);
    comm.collective(std::move(a), req);
  }
  static void run_allreduce(internal::Resolved&& r, comm_type& comm, req_type* req, HostAlgo) {
    run(std::move(r), comm, req);
  }
  using p2p_item = internal::host::P2PItem;
  static p2p_item make_send(const void* buf, size_t bytes, int peer) {
    p2p_item it; it.is_send = true; it.peer = peer; it.sbuf = buf; it.bytes = bytes; return it;
  }
  static p2p_item make_recv(void* buf, size_t bytes, int peer) {
    p2p_item it; it.is_send = false; it.peer = peer; it.rbuf = buf; it.bytes = bytes; return it;
  }
  static void run_p2p(std::vector<internal::host::P2PItem>&& items, comm_type& comm, req_type* req, const char* name) {
    comm.p2p(std::move(items), req, name);
  }
  static bool test(req_type& req) {
    if (!req) return true;
    const int s = req->status.load(std::memory_order_acquire);
    if (s == 0) return false;
    req_type done = std::move(req);
    req = nullptr;
    if (s == 2) throw_al_exception(done->error);
    return true;
  }
  static void wait(req_type& req) {
    if (!req) return;
    unsigned spins = 0;
    while (req->status.load(std::memory_order_acquire) == 0) {
      if (++spins > 200) std::this_thread::yield();
    }
    (void)test(req);
  }
  static void register_memory(void*, size_t, comm_type&) {}
  static void unregister_memory(void*, comm_type&) {}
};

}  // namespace Al
