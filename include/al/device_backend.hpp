/**
 * @file device_backend.hpp
 * The GPU backend: every operation is one hand-written sm_100a kernel working
 * directly in peer GPUs' memory over NVLink (see al/device/params.hpp for the
 * protocol).  It fills the role of Al::NCCLBackend
 * (include/aluminum/nccl_impl.hpp:299-1431) without calling NCCL.
 *
 * Completion semantics are the reference's (nccl_impl.hpp:902-940,1406-1429):
 *   blocking      enqueued on the communicator's stream, host returns at once;
 *   non-blocking  enqueued on a pooled high-priority stream that first waits
 *                 for the communicator's stream; the request carries an event;
 *   Wait(req)     makes the communicator's stream wait for the event (host
 *                 does not block) and - unlike the reference - resets req;
 *   Test(req)     host-side poll, resets req when complete.
 * With AL_REQ_MEMOPS=1 the event is replaced by a pinned flag written with
 * cuStreamWriteValue32 and awaited with cuStreamWaitValue32, so Test is a
 * plain host load and Wait involves no event.
 */
#pragma once
#include <atomic>
#include <mutex>
#include <string>

#include "al/cuda/events.hpp"
#include "al/cuda/streams.hpp"
#include "al/cuda/sync_memory.hpp"
#include "al/device/communicator.hpp"
#include "al/resolve.hpp"
#include "al/tuning.hpp"

namespace Al {

namespace internal {
namespace device {

/** First failure of a communicator's background operations, shared with the requests they returned. */
struct AsyncFailure {
  std::atomic<bool> failed{false};
  std::mutex mu;
  std::string message;
  void set(const std::string& what) {
    std::lock_guard<std::mutex> lock(mu);
    if (!failed.load()) { message = what; failed.store(true, std::memory_order_release); }
  }
  /** Throws al_exception if a failure was recorded. */
  void check(const char* context) {
    if (!failed.load(std::memory_order_acquire)) return;
    std::lock_guard<std::mutex> lock(mu);
    throw_al_exception(context, ": ", message);
  }
};

struct RequestState {
  cudaEvent_t event = nullptr;      // event mode
  int32_t* flag = nullptr;          // memops mode: the internal stream's pinned counter word (not owned)
  CUdeviceptr flag_dev = 0;
  uint32_t ticket = 0;              // memops mode: complete once the counter reached this value
  cudaStream_t orig_stream = nullptr;
  cudaStream_t internal_stream = nullptr;
  std::shared_ptr<DeviceCommunicator::Impl> comm;
  std::shared_ptr<AsyncFailure> failure;  // host-transfer operations: where the progress engine reports errors
  ~RequestState() {
    if (event) cuda::event_pool.release(event);
  }
};
using Request = std::shared_ptr<RequestState>;

/** Internal stream for a non-blocking operation, already ordered after `comm`'s stream. */
cudaStream_t begin_nonblocking(DeviceCommunicator& comm);
/** Record completion on `internal_stream` and build the request. */
Request end_nonblocking(DeviceCommunicator& comm, cudaStream_t internal_stream);
cudaStream_t begin_nonblocking_stream(cudaStream_t comm_stream);
/** The same with a given internal stream instead of one from the pool. */
cudaStream_t begin_nonblocking_on(cudaStream_t comm_stream, cudaStream_t internal);
/** A new highest-priority, non-blocking stream (the caller destroys it). */
cudaStream_t create_internal_stream();
Request end_nonblocking_stream(cudaStream_t comm_stream, cudaStream_t internal_stream);
bool test_request(Request& req);
void wait_request(Request& req);

}  // namespace device
}  // namespace internal

using DeviceAllreduceAlgo = internal::device::AllreduceAlgo;
/** `algo` argument of every device collective but allreduce: automatic, staged or window (see CollPath). */
using DeviceAlgo = internal::device::CollPath;

class DeviceBackend {
 public:
  using comm_type = DeviceCommunicator;
  using req_type = internal::device::Request;
  static constexpr std::nullptr_t null_req = nullptr;
  using allreduce_algo_type = DeviceAllreduceAlgo;  using reduce_algo_type = DeviceAlgo;
  using reduce_scatter_algo_type = DeviceAlgo;  using reduce_scatterv_algo_type = DeviceAlgo;
  using allgather_algo_type = DeviceAlgo;  using allgatherv_algo_type = DeviceAlgo;
  using alltoall_algo_type = DeviceAlgo;  using alltoallv_algo_type = DeviceAlgo;
  using barrier_algo_type = DeviceAlgo;  using bcast_algo_type = DeviceAlgo;
  using gather_algo_type = DeviceAlgo;  using gatherv_algo_type = DeviceAlgo;
  using scatter_algo_type = DeviceAlgo;  using scatterv_algo_type = DeviceAlgo;
  static std::string Name() { return "DeviceBackend"; }

  static void run(internal::Resolved&& r, comm_type& comm, req_type* req, int path = 0,
                  DeviceAllreduceAlgo algo = DeviceAllreduceAlgo::automatic) {
    using namespace internal::device;
    ScopedDevice on_device(comm.device());
    CollDesc d;
    d.kind = (DevColl)(int)r.kind;
    d.in = d.wire = d.out = r.dt;
    d.op = r.op; d.root = r.root; d.count = r.count; d.vector = r.vector; d.algo = algo;
    d.path = (CollPath)path;
    std::vector<RankArgs> ra(1);
    ra[0].send = r.send; ra[0].recv = r.recv;
    ra[0].send_counts = std::move(r.send_counts); ra[0].send_displs = std::move(r.send_displs);
    ra[0].recv_counts = std::move(r.recv_counts); ra[0].recv_displs = std::move(r.recv_displs);
    if (req) {
      cudaStream_t s = begin_nonblocking(comm);
      comm.collective(d, ra, s);
      *req = end_nonblocking(comm, s);
    } else {
      comm.collective(d, ra, comm.get_stream());
    }
  }
  static void run_allreduce(internal::Resolved&& r, comm_type& comm, req_type* req, DeviceAllreduceAlgo algo) {
    run(std::move(r), comm, req, 0, algo);
  }
  using p2p_item = internal::device::P2PDesc;
  static p2p_item make_send(const void* buf, size_t bytes, int peer) {
    p2p_item it; it.is_send = true; it.peer = peer; it.sbuf = buf; it.bytes = bytes; return it;
  }
  static p2p_item make_recv(void* buf, size_t bytes, int peer) {
    p2p_item it; it.is_send = false; it.peer = peer; it.rbuf = buf; it.bytes = bytes; return it;
  }
  static void run_p2p(std::vector<internal::device::P2PDesc>&& items, comm_type& comm, req_type* req, const char*) {
    using namespace internal::device;
    ScopedDevice on_device(comm.device());
    if (req) {
      cudaStream_t s = begin_nonblocking(comm);
      comm.p2p(items, s);
      *req = end_nonblocking(comm, s);
    } else {
      comm.p2p(items, comm.get_stream());
    }
  }
  static bool test(req_type& req) { return internal::device::test_request(req); }
  static void wait(req_type& req) { internal::device::wait_request(req); }
  /**
   * Collective over the communicator (every rank calls it, in the same order, with its own buffer):
   * the buffer becomes addressable by every rank, and reduce_scatter / allgather / alltoall / bcast on
   * it skip the staging area.  Role of ncclCommRegister in the reference (src/nccl_impl.cpp:83-109),
   * which is a local call there; buffers from comm.symm_alloc() need no registration.
   */
  static void register_memory(void* buf, size_t bytes, comm_type& comm) { (void)comm.register_buffer(buf, bytes); }
  static void unregister_memory(void* buf, comm_type& comm) { comm.unregister_buffer(buf); }
};

}  // namespace Al
