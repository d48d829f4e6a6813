// Private to the host backend's translation units: the communicator's state
// shared by the shared-memory path (host_comm.cpp) and the socket path
// (host_net.cpp), and the base class of their progress-engine states.
#pragma once
#include <atomic>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "al/host/communicator.hpp"
#include "al/mempool.hpp"
#include "al/state.hpp"
#include "al/tuning.hpp"
#include "al/util/utils.hpp"

#if defined(__x86_64__)
#include <immintrin.h>
#define AL_CPU_RELAX() _mm_pause()
#else
#define AL_CPU_RELAX() ((void)0)
#endif

namespace Al {
namespace internal {
namespace host {
class Workspace;  // shared-memory segment of a single-node communicator (host_comm.cpp)
class NetMesh;    // sockets of a communicator that spans nodes (host_net.cpp)
}  // namespace host
}  // namespace internal

struct HostCommunicator::Impl {
  std::unique_ptr<internal::host::Workspace> ws;   // single node
  std::unique_ptr<internal::host::NetMesh> net;    // several nodes (exactly one of the two is set)
  // Two-level layout of a communicator that spans nodes and has a node with several members:
  // a shared-memory communicator per node and a socket communicator of the nodes' first members.
  std::unique_ptr<HostCommunicator> node_comm, leader_comm;  // leader_comm only on the first member of a node
  // When every node holds the same number of members: the members with equal node-local rank, one per node.
  std::unique_ptr<HostCommunicator> rail_comm;
  std::vector<int> node_of;       // member -> index of its node (nodes numbered by their lowest member)
  std::vector<int> local_index;   // member -> rank inside its node's communicator
  int p = 1, me = 0;
  internal::World* world = nullptr;
  std::vector<int> world_rank_of;      // member -> world rank (for liveness checks and messages)
  std::atomic<uint64_t> next_seq{1};   // collective sequence numbers handed out at call time
  std::atomic<uint64_t> done_seq{0};   // last collective that finished locally
  std::vector<std::atomic<uint64_t>> send_next, send_serving, recv_next, recv_serving;
  std::atomic<bool> failed{false};
  std::atomic<uint64_t> n_coll{0}, n_p2p{0}, n_bytes{0}, n_fail{0};
  std::string fail_msg;
  std::mutex fail_mu;
  // Local shadows of the mailbox counters this rank owns as a writer.
  std::vector<uint64_t> sent_count, acked_count;

  explicit Impl(const internal::Group& g);
  ~Impl();
  /**
   * Record the first failure and tell the peers: a word in the shared workspace (single node) or a
   * shutdown of this communicator's connections (several nodes) ends their waits at once, and the
   * node / leader / rail communicators of a two-level layout are failed along with their parent.
   */
  void fail(const std::string& msg);
  /** Member rank + 1 of a peer that failed this (single-node) communicator, 0 if none has. */
  uint64_t poisoned_by() const;
};

namespace internal {
namespace host {

/** Base of host states: owns the request and the time-out bookkeeping. */
class HostState : public AlState {
 public:
  HostState(HostCommunicator::Impl* ci, Request req) : ci_(ci), req_(std::move(req)) {}
  ~HostState() override {
    for (void* t : temps_) mempool.release_bytes(MemoryType::HOST, t);
  }
  const void* get_compute_stream() const override { return ci_; }
  /** Keep a host buffer from the memory pool alive until the state is destroyed. */
  void adopt_temp(void* t) { temps_.push_back(t); }
  /** A pooled host buffer that lives as long as the state. */
  void* temp(size_t bytes) {
    void* t = mempool.allocate_bytes(MemoryType::HOST, bytes ? bytes : 1);
    temps_.push_back(t);
    return t;
  }

 protected:
  /** Returns true (and records the failure) when the current wait exceeded the limit. */
  bool timed_out(const char* what) {
    if (ci_->failed.load(std::memory_order_acquire) && !failed_) {
      fail("communicator failed: " + ci_->fail_msg);
      return true;
    }
    if (const uint64_t by = ci_->poisoned_by()) {
      fail(build_string(get_name(), ": rank ", by - 1, " reported a failure on this communicator"));
      return true;
    }
    const double now = get_time();
    if (wait_since_ == 0) { wait_since_ = now; return false; }
    if (now - wait_since_ > tuning().host_wait_timeout_s) {
      fail(build_string(get_name(), ": timed out after ", tuning().host_wait_timeout_s, " s waiting for ", what));
      return true;
    }
    return false;
  }
  void progress_made() { wait_since_ = 0; }
  /**
   * While waiting for member `r`: has its process gone?  Looks at the control
   * connection at most every 50 ms.  A rank that exited can never arrive, so
   * the caller fails at once instead of sitting out the time-out.
   */
  bool peer_gone(int r) {
    const double now = get_time();
    if (now - last_alive_check_ < 0.05 && r == last_alive_rank_) return false;
    last_alive_check_ = now;
    last_alive_rank_ = r;
    return ci_->world && !ci_->world->peer_alive(ci_->world_rank_of[(size_t)r]);
  }
  double last_alive_check_ = 0;
  int last_alive_rank_ = -1;
  // The outcome reaches the request only in publish_outcome(), the last thing a
  // state does: once the request is complete its owner may destroy the
  // communicator, so nothing of *ci_ may be touched afterwards.
  void fail(const std::string& msg) {
    ci_->fail(msg);
    ci_->n_fail.fetch_add(1, std::memory_order_relaxed);
    err_ = msg;
    failed_ = true;
  }
  void publish_outcome() {
    if (!req_ || published_) return;
    published_ = true;
    if (failed_) {
      req_->error = err_;
      req_->status.store(2, std::memory_order_release);
    } else {
      req_->status.store(1, std::memory_order_release);
    }
  }
  std::string err_;
  bool published_ = false;
  std::vector<void*> temps_;
  HostCommunicator::Impl* ci_;
  Request req_;
  double wait_since_ = 0;
  bool failed_ = false;

 public:
  bool has_failed() const { return failed_; }
};


/** Drive a state on the calling thread until it completes. */
template <typename State>
void run_inline(State& st) {
  st.start();
  unsigned spins = 0;
  while (st.step() != PEAction::complete) {
    if (++spins < 200) AL_CPU_RELAX();
    else std::this_thread::yield();
  }
}

/** The state that runs `args` on communicator `ci`: two-level, socket or shared-memory path (host_comm.cpp). */
HostState* make_collective_state(HostCommunicator::Impl* ci, CollArgs&& args, Request req, uint64_t seq);
/** Allreduce / bcast / barrier composed of node-level and leader-level operations (host_hier.cpp); nullptr if not applicable. */
HostState* make_hier_collective(HostCommunicator::Impl* ci, CollArgs& args, Request req, uint64_t seq);

/** States of the socket path (host_net.cpp). */
HostState* make_net_collective(HostCommunicator::Impl* ci, CollArgs&& args, Request req, uint64_t seq);
HostState* make_net_p2p(HostCommunicator::Impl* ci, std::vector<P2PItem>&& items, Request req, const char* name);

}  // namespace host
}  // namespace internal
}  // namespace Al
