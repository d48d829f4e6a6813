// Host-transfer backend: staging copies, flags and the engine state (see al/ht_backend.hpp).
#include "al/ht_backend.hpp"

#include <algorithm>
#include <cstring>

#include "al/cuda/gpu_status_flag.hpp"
#include "al/cuda/gpu_wait.hpp"
#include "al/mempool.hpp"
#include "al/progress.hpp"
#include "al/runtime.hpp"

namespace Al {
namespace internal {
namespace ht {

namespace {

/** Engine state shared by collectives and point-to-point: stage 0 waits for the D2H flag. */
class HTState final : public AlState {
 public:
  HTState(cudaStream_t stream, const char* name, std::shared_ptr<device::AsyncFailure> failure)
      : failure_(std::move(failure)), stream_(stream), name_(name) {}
  ~HTState() override {
    for (void* p : pinned_) mempool.release_bytes(MemoryType::CUDA_PINNED_HOST, p);
  }
  const void* get_compute_stream() const override { return stream_; }
  const char* get_name() const override { return name_; }
  RunType get_run_type() const override { return unbounded_ ? RunType::unbounded : RunType::bounded; }

  PEAction step() override {
    switch (phase_) {
      case 0:
        if (!start_flag.query()) return PEAction::cont;
        phase_ = 1;
        return PEAction::advance;
      case 1:
        try {
          launch_host();  // non-blocking host operation driven by the same engine
        } catch (const std::exception& e) {
          // The host communicator refused the operation (it failed earlier): release the
          // stream so that nothing on the device waits forever, and say why.
          // The failure is recorded BEFORE the stream is released, so whoever sees the operation's
          // completion event also sees the error.
          failure_->set(std::string("the host exchange could not start: ") + e.what());
          poison_receive_buffers();
          wait.signal();
          phase_ = 3;
          return PEAction::cont;
        }
        // A rank that receives nothing (non-root of reduce / gather, root of
        // scatter with no slice, a pure send) only had to get its data off the
        // device: its stream is released now instead of after the exchange
        // (the reference signals such ranks early too, e.g.
        // include/aluminum/ht/reduce.hpp and ht/gather.hpp).
        if (early_release_) wait.signal();
        phase_ = 2;
        return PEAction::cont;
      case 2:
        try {
          if (!HostBackend::test(host_req)) return PEAction::cont;
        } catch (const std::exception& e) {
          failure_->set(e.what());
          poison_receive_buffers();
        }
        if (!early_release_) wait.signal();  // release the stream: H2D copy and end flag follow
        phase_ = 3;
        return PEAction::cont;
      default:
        if (!end_flag.query()) return PEAction::cont;
        // Only the spin-kernel fallback of the stream's wait has a time budget; if it ran out, the stream copied
        // the receive buffers back before the exchange had filled them.
        if (wait.timed_out())
          failure_->set("the stream stopped waiting for the host exchange (device wait time-out); the result is not valid");
        return PEAction::complete;
    }
  }

  void* pinned(size_t bytes) {
    void* p = mempool.allocate_bytes(MemoryType::CUDA_PINNED_HOST, std::max<size_t>(bytes, 1));
    pinned_.push_back(p);
    return p;
  }
  /** Host buffers whose contents go back to the device when the stream is released. */
  void returns_to_device(void* host, size_t bytes) { back_.push_back({host, bytes}); }

  cuda::GPUStatusFlag start_flag, end_flag;
  cuda::GPUWait wait;
  HostBackend::req_type host_req;
  std::function<void(HostBackend::req_type*)> launcher;
  bool unbounded_ = false;
  bool early_release_ = false;  ///< nothing comes back to the device: do not hold the stream during the exchange

 private:
  void launch_host() { launcher(&host_req); }
  /**
   * The copies back to the device are already enqueued behind the stream's wait and cannot be
   * withdrawn; after a failure they carry 0xFF bytes (NaN for floating-point types) instead of
   * stale pool memory, so a result that is used in spite of the error is conspicuous.
   */
  void poison_receive_buffers() {
    for (auto& b : back_) memset(b.first, 0xFF, b.second);
  }
  std::shared_ptr<device::AsyncFailure> failure_;
  std::vector<std::pair<void*, size_t>> back_;
  cudaStream_t stream_;
  const char* name_;
  int phase_ = 0;
  std::vector<void*> pinned_;
};

}  // namespace

void run_collective(Resolved&& r, HostTransferCommunicator& comm, cudaStream_t stream) {
  const Extent e = extent_of(r, comm.rank(), comm.size());
  const size_t esz = dtype_size(r.dt);
  comm.failure()->check("host-transfer communicator failed earlier");
  auto* st = new HTState(stream, "HTCollective", comm.failure());
  void* hsend = e.send_elems ? st->pinned(e.send_elems * esz) : nullptr;
  void* hrecv = e.recv_elems ? st->pinned(e.recv_elems * esz) : nullptr;
  const void* dsend = r.send;
  void* drecv = r.recv;
  if (hsend) AL_CHECK_CUDA(cudaMemcpyAsync(hsend, dsend, e.send_elems * esz, cudaMemcpyDeviceToHost, stream));
  // Vector forms may leave gaps in the receive buffer: start from its current contents.
  if (hrecv && r.vector) AL_CHECK_CUDA(cudaMemcpyAsync(hrecv, drecv, e.recv_elems * esz, cudaMemcpyDeviceToHost, stream));
  st->start_flag.record(stream);
  st->wait.wait(stream);
  if (hrecv) {
    AL_CHECK_CUDA(cudaMemcpyAsync(drecv, hrecv, e.recv_elems * esz, cudaMemcpyHostToDevice, stream));
    st->returns_to_device(hrecv, e.recv_elems * esz);
  }
  st->end_flag.record(stream);
  st->early_release_ = hrecv == nullptr && r.kind != OpKind::barrier;  // a barrier holds the stream by definition

  auto shared = std::make_shared<Resolved>(std::move(r));
  shared->send = hsend;
  shared->recv = hrecv;
  if (shared->kind == OpKind::bcast) { shared->send = shared->recv = hsend ? hsend : hrecv; }
  HostCommunicator* hc = &comm.host();
  st->launcher = [shared, hc](HostBackend::req_type* req) {
    Resolved copy = *shared;
    HostBackend::run(std::move(copy), *hc, req);
  };
  get_progress_engine()->enqueue(st);
}

void run_p2p(std::vector<host::P2PItem>&& items, HostTransferCommunicator& comm, cudaStream_t stream, const char* name) {
  comm.failure()->check("host-transfer communicator failed earlier");
  auto* st = new HTState(stream, name, comm.failure());
  st->unbounded_ = true;
  struct Back { void* host; void* dev; size_t bytes; };
  std::vector<Back> backs;
  for (auto& it : items) {
    if (it.is_send) {
      void* h = st->pinned(it.bytes);
      if (it.bytes) AL_CHECK_CUDA(cudaMemcpyAsync(h, it.sbuf, it.bytes, cudaMemcpyDeviceToHost, stream));
      it.sbuf = h;
    } else {
      void* h = st->pinned(it.bytes);
      backs.push_back({h, it.rbuf, it.bytes});
      it.rbuf = h;
    }
  }
  st->start_flag.record(stream);
  st->wait.wait(stream);
  for (auto& b : backs) {
    if (b.bytes) AL_CHECK_CUDA(cudaMemcpyAsync(b.dev, b.host, b.bytes, cudaMemcpyHostToDevice, stream));
    st->returns_to_device(b.host, b.bytes);
  }
  st->end_flag.record(stream);
  st->early_release_ = backs.empty();
  auto shared = std::make_shared<std::vector<host::P2PItem>>(std::move(items));
  HostCommunicator* hc = &comm.host();
  st->launcher = [shared, hc, name](HostBackend::req_type* req) {
    std::vector<host::P2PItem> copy = *shared;
    HostBackend::run_p2p(std::move(copy), *hc, req, name);
  };
  get_progress_engine()->enqueue(st);
}

}  // namespace ht
}  // namespace internal
}  // namespace Al
