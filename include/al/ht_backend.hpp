/**
 * @file ht_backend.hpp
 * Host-transfer backend: GPU buffers are staged through pinned host memory
 * and the operation itself runs between CPU ranks.  It is the fallback for
 * buffers or systems where peer mapping is unavailable, and it exercises the
 * progress engine together with the stream write/wait-value flags.
 *
 * Parity: Al::HostTransferBackend (include/aluminum/ht_impl.hpp,
 * include/aluminum/ht/base_state.hpp:41-209, e.g. ht/allreduce.hpp:41-79).
 * Flow of every operation, all enqueued at call time:
 *   D2H copies -> GPUStatusFlag.record (tells the engine the data landed)
 *   -> GPUWait.wait (stream stalls) -> H2D copy -> GPUStatusFlag.record.
 * The engine state waits for the first flag in pipeline stage 0, advances,
 * runs the host operation, signals the GPUWait and completes when the second
 * flag fires.  A rank that receives nothing back (non-root of reduce / gather,
 * a pure send) is signalled as soon as its data has left the device, like the
 * reference's early-signalling policies (ht/base_state.hpp:86-209); every
 * other rank when the host exchange is complete.
 */
#pragma once
#include <memory>

#include "al/device_backend.hpp"
#include "al/host_backend.hpp"
#include "al/progress.hpp"

namespace Al {

class HostTransferCommunicator {
 public:
  HostTransferCommunicator() : HostTransferCommunicator((cudaStream_t) nullptr) {}
  explicit HostTransferCommunicator(cudaStream_t stream)
      : host_(), stream_(stream), failure_(std::make_shared<internal::device::AsyncFailure>()) {}
  HostTransferCommunicator(const internal::Group& g, cudaStream_t stream)
      : host_(g), stream_(stream), failure_(std::make_shared<internal::device::AsyncFailure>()) {}
  HostTransferCommunicator(HostTransferCommunicator&&) noexcept = default;
  HostTransferCommunicator& operator=(HostTransferCommunicator&&) noexcept = default;
  HostTransferCommunicator copy(cudaStream_t stream = nullptr) const {
    return HostTransferCommunicator(host_.group(), stream);
  }
  /** MPI_Comm_split analogue (collective). */
  HostTransferCommunicator split(int color, int key, cudaStream_t stream = nullptr) const {
    return HostTransferCommunicator(host_.group().split(color, key), stream);
  }
  int rank() const { return host_.rank(); }
  int size() const { return host_.size(); }
  int local_rank() const { return host_.local_rank(); }
  int local_size() const { return host_.local_size(); }
  cudaStream_t get_stream() const { return stream_; }
  HostCommunicator& host() { return host_; }
  /**
   * Where the progress engine records a failed host exchange (a peer that exited, a time-out,
   * abort).  Once set, every later call on this communicator and Test / Wait on its requests
   * throw; the device buffers of the failed operation hold no valid result.
   */
  const std::shared_ptr<internal::device::AsyncFailure>& failure() const { return failure_; }
  bool failed() const { return failure_->failed.load(std::memory_order_acquire); }
  /**
   * The stream non-blocking operations of this communicator run on, created
   * on first use.  Every host-transfer communicator has its own: an operation
   * holds its stream until the host exchange is complete, so operations of
   * different communicators must never queue behind one another - two ranks
   * whose threads reach a shared stream in different orders would wait for
   * each other forever.  (The reference shares its pooled internal streams.)
   */
  cudaStream_t internal_stream() {
    if (!internal_) {
      internal_ = std::shared_ptr<CUstream_st>(internal::device::create_internal_stream(),
                                               [](cudaStream_t s) {
                                                 internal::release_progress_key(s);
                                                 (void)cudaStreamDestroy(s);
                                               });
    }
    return internal_.get();
  }

 private:
  HostCommunicator host_;
  cudaStream_t stream_;
  std::shared_ptr<internal::device::AsyncFailure> failure_;
  std::shared_ptr<CUstream_st> internal_;
};

namespace internal {
namespace ht {
/** Enqueue the staging copies and flags on `stream` and hand the operation to the progress engine. */
void run_collective(Resolved&& r, HostTransferCommunicator& comm, cudaStream_t stream);
void run_p2p(std::vector<host::P2PItem>&& items, HostTransferCommunicator& comm, cudaStream_t stream, const char* name);
}  // namespace ht
}  // namespace internal

class HostTransferBackend {
 public:
  using comm_type = HostTransferCommunicator;
  using req_type = internal::device::Request;
  static constexpr std::nullptr_t null_req = nullptr;
  using allreduce_algo_type = HostAlgo;  using reduce_algo_type = HostAlgo;
  using reduce_scatter_algo_type = HostAlgo;  using reduce_scatterv_algo_type = HostAlgo;
  using allgather_algo_type = HostAlgo;  using allgatherv_algo_type = HostAlgo;
  using alltoall_algo_type = HostAlgo;  using alltoallv_algo_type = HostAlgo;
  using barrier_algo_type = HostAlgo;  using bcast_algo_type = HostAlgo;
  using gather_algo_type = HostAlgo;  using gatherv_algo_type = HostAlgo;
  using scatter_algo_type = HostAlgo;  using scatterv_algo_type = HostAlgo;
  static std::string Name() { return "HostTransferBackend"; }

  static void run(internal::Resolved&& r, comm_type& comm, req_type* req, int /*algo*/ = 0) {
    using namespace internal::device;
    if (req) {
      cudaStream_t s = begin_nonblocking_on(comm.get_stream(), comm.internal_stream());
      internal::ht::run_collective(std::move(r), comm, s);
      *req = end_nonblocking_stream(comm.get_stream(), s);
      (*req)->failure = comm.failure();
    } else {
      internal::ht::run_collective(std::move(r), comm, comm.get_stream());
    }
  }
  static void run_allreduce(internal::Resolved&& r, comm_type& comm, req_type* req, HostAlgo) {
    run(std::move(r), comm, req);
  }
  using p2p_item = internal::host::P2PItem;
  static p2p_item make_send(const void* buf, size_t bytes, int peer) { return HostBackend::make_send(buf, bytes, peer); }
  static p2p_item make_recv(void* buf, size_t bytes, int peer) { return HostBackend::make_recv(buf, bytes, peer); }
  static void run_p2p(std::vector<p2p_item>&& items, comm_type& comm, req_type* req, const char* name) {
    using namespace internal::device;
    if (req) {
      cudaStream_t s = begin_nonblocking_on(comm.get_stream(), comm.internal_stream());
      internal::ht::run_p2p(std::move(items), comm, s, name);
      *req = end_nonblocking_stream(comm.get_stream(), s);
      (*req)->failure = comm.failure();
    } else {
      internal::ht::run_p2p(std::move(items), comm, comm.get_stream(), name);
    }
  }
  static bool test(req_type& req) { return internal::device::test_request(req); }
  static void wait(req_type& req) { internal::device::wait_request(req); }
  static void register_memory(void*, size_t, comm_type&) {}
  static void unregister_memory(void*, comm_type&) {}
};

}  // namespace Al
