// Non-blocking plumbing of the device backend (see al/device_backend.hpp).
#include "al/device_backend.hpp"
#include "al/util/utils.hpp"

#include <mutex>
#include <vector>

namespace Al {
namespace internal {
namespace device {

namespace {
bool use_memops() {
  static const bool v = env_long("AL_REQ_MEMOPS", 0) != 0;
  return v && cuda::stream_memory_operations_supported();
}
}  // namespace

cudaStream_t begin_nonblocking(DeviceCommunicator& comm) { return begin_nonblocking_stream(comm.get_stream()); }

cudaStream_t begin_nonblocking_stream(cudaStream_t comm_stream) {
  if (tuning().disable_background_streams) return comm_stream;
  return begin_nonblocking_on(comm_stream, cuda::stream_pool.get_high_priority_stream());
}

cudaStream_t create_internal_stream() {
  int least = 0, greatest = 0;
  AL_CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&least, &greatest));
  cudaStream_t s = nullptr;
  AL_CHECK_CUDA(cudaStreamCreateWithPriority(&s, cudaStreamNonBlocking, greatest));
  return s;
}

cudaStream_t begin_nonblocking_on(cudaStream_t comm_stream, cudaStream_t internal) {
  if (tuning().disable_background_streams) return comm_stream;
  cudaEvent_t ev = cuda::event_pool.get();
  AL_CHECK_CUDA(cudaEventRecord(ev, comm_stream));
  AL_CHECK_CUDA(cudaStreamWaitEvent(internal, ev, 0));
  cuda::event_pool.release(ev);  // the wait has captured the event's current record
  return internal;
}

namespace {
// Memops mode: one pinned counter word per internal stream.  Operation number t
// on that stream writes t when it completes; waiting means "counter >= t"
// (cyclic comparison), so words are never reset or recycled.
struct StreamCounter { int32_t* word = nullptr; CUdeviceptr dev = 0; uint32_t next = 0; };
std::mutex g_ctr_mu;
std::vector<std::pair<cudaStream_t, StreamCounter>> g_counters;

StreamCounter& counter_for(cudaStream_t s) {
  for (auto& kv : g_counters)
    if (kv.first == s) return kv.second;
  StreamCounter c;
  c.word = cuda::sync_pool.get();
  __atomic_store_n(c.word, 0, __ATOMIC_SEQ_CST);
  void* dp = nullptr;
  AL_CHECK_CUDA(cudaHostGetDevicePointer(&dp, c.word, 0));
  c.dev = (CUdeviceptr)dp;
  g_counters.emplace_back(s, c);
  return g_counters.back().second;
}
}  // namespace

Request end_nonblocking(DeviceCommunicator& comm, cudaStream_t internal_stream) {
  return end_nonblocking_stream(comm.get_stream(), internal_stream);
}

Request end_nonblocking_stream(cudaStream_t comm_stream, cudaStream_t internal_stream) {
  Request req = std::make_shared<RequestState>();
  req->orig_stream = comm_stream;
  req->internal_stream = internal_stream;
  if (use_memops()) {
    std::lock_guard<std::mutex> g(g_ctr_mu);
    StreamCounter& c = counter_for(internal_stream);
    req->flag = c.word;
    req->flag_dev = c.dev;
    req->ticket = ++c.next;
    AL_CHECK_CUDA_DRV(cuda::drv().StreamWriteValue32((CUstream)internal_stream, c.dev, req->ticket, CU_STREAM_WRITE_VALUE_DEFAULT));
  } else {
    req->event = cuda::event_pool.get();
    AL_CHECK_CUDA(cudaEventRecord(req->event, internal_stream));
  }
  return req;
}

bool test_request(Request& req) {
  if (!req) return true;
  if (req->failure) req->failure->check("host-transfer operation failed");
  bool done;
  if (req->flag) {
    done = (int32_t)((uint32_t)__atomic_load_n(req->flag, __ATOMIC_ACQUIRE) - req->ticket) >= 0;
  } else {
    cudaError_t e = cudaEventQuery(req->event);
    if (e == cudaErrorNotReady) { (void)cudaGetLastError(); done = false; }
    else { AL_CHECK_CUDA(e); done = true; }
  }
  if (done) {
    // the host side of a host-transfer operation reports before it releases the stream
    if (req->failure) req->failure->check("host-transfer operation failed");
    req = nullptr;
  }
  return done;
}

void wait_request(Request& req) {
  if (!req) return;
  if (req->failure) req->failure->check("host-transfer operation failed");
  if (req->internal_stream != req->orig_stream) {
    if (req->flag)
      AL_CHECK_CUDA_DRV(cuda::drv().StreamWaitValue32((CUstream)req->orig_stream, req->flag_dev, req->ticket, CU_STREAM_WAIT_VALUE_GEQ));
    else
      AL_CHECK_CUDA(cudaStreamWaitEvent(req->orig_stream, req->event, 0));
  }
  req = nullptr;  // the enqueued wait holds everything it needs
}

}  // namespace device
}  // namespace internal
}  // namespace Al
