// Host (shared-memory) backend: workspace, collective and point-to-point state
// machines.  See al/host/communicator.hpp for the role of this backend.
//
// Protocol (shared with the device kernels):
//   * every rank owns a region of the communicator's shared segment holding two
//     staging halves, per-source epoch flags A/B/C, a per-source "meta" word
//     and one two-slot mailbox per source rank for point-to-point traffic;
//   * a collective with sequence number k runs in G chunks.  In chunk c every
//     rank copies ("publishes") its contribution into staging half (k+c)&1,
//     then stores the epoch (k<<24 | c+1) into flag A[me] of every rank, then
//     waits until all of its own A flags reached that epoch, then pulls or
//     reduces from the peers' staging.  Two-phase ops (allreduce) repeat the
//     handshake with the B flags.  Because every chunk of every op makes every
//     rank wait for every other rank, a rank that publishes chunk c+2 knows
//     that all peers finished reading chunk c: two halves suffice.
//   * G is the maximum over ranks of the chunk count each rank needs, exchanged
//     through the meta words together with the first A flag, so ranks need not
//     know each other's counts in vector operations.
#include "al/host/communicator.hpp"

#include "host_impl.hpp"
#include "host_net.hpp"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <random>
#include <thread>

#include "al/host/reduce.hpp"
#include "al/mempool.hpp"
#include "al/progress.hpp"
#include "al/runtime.hpp"
#include "al/state.hpp"
#include "al/trace.hpp"
#include "al/tuning.hpp"
#include "al/util/meta.hpp"
#include "al/util/utils.hpp"

namespace Al {
namespace internal {
namespace host {

using flag_t = std::atomic<uint64_t>;
static_assert(sizeof(flag_t) == 8, "flags are shared between processes as plain 8-byte words");

constexpr size_t kLine = 64;

/** Byte offsets inside one rank's region. */
struct Layout {
  int p = 1;
  size_t half = 0, slot = 0;
  size_t off_A = 0, off_B = 0, off_C = 0, off_meta = 0, off_mctl = 0, off_poison = 0, off_stage = 0, off_mbox = 0, region = 0;
  Layout() = default;
  Layout(int p_, size_t half_, size_t slot_) : p(p_), half(half_), slot(round_up(slot_, kLine)) {
    size_t o = 0;
    off_A = o; o += (size_t)p * kLine;
    off_B = o; o += (size_t)p * kLine;
    off_C = o; o += (size_t)p * kLine;
    off_meta = o; o += 2 * (size_t)p * kLine;
    off_mctl = o; o += 2 * (size_t)p * kLine;  // sent, acked per source
    off_poison = o; o += kLine;                // only the word in region 0 is used
    o = round_up(o, 4096);
    off_stage = o; o += 2 * half;
    off_mbox = o; o += (size_t)p * 2 * slot;
    region = round_up(o, 4096);
  }
};

class Workspace {
 public:
  Workspace(const Group& g, uint64_t id, size_t half, size_t slot) : lay_(g.size(), half, slot) {
    name_ = "/al_b200_" + std::to_string((unsigned long long)std::hash<std::string>{}(g.world()->job_key())) +
            "_" + std::to_string((unsigned long long)id);
    bytes_ = lay_.region * (size_t)g.size();
    int fd = -1;
    if (g.rank() == 0) {
      shm_unlink(name_.c_str());
      fd = shm_open(name_.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
      if (fd < 0) throw_al_exception("shm_open(create ", name_, "): ", strerror(errno));
      if (ftruncate(fd, (off_t)bytes_) != 0) throw_al_exception("ftruncate: ", strerror(errno));
    }
    g.barrier();
    if (g.rank() != 0) {
      fd = shm_open(name_.c_str(), O_RDWR, 0600);
      if (fd < 0) throw_al_exception("shm_open(", name_, "): ", strerror(errno));
    }
    base_ = (char*)mmap(nullptr, bytes_, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (base_ == MAP_FAILED) throw_al_exception("mmap of shared workspace failed: ", strerror(errno));
    g.barrier();  // everyone has mapped: the name can go (fresh pages are zero = epoch 0)
    if (g.rank() == 0) shm_unlink(name_.c_str());
  }
  ~Workspace() {
    if (base_ && base_ != MAP_FAILED) munmap(base_, bytes_);
  }
  const Layout& lay() const { return lay_; }
  char* region(int r) const { return base_ + lay_.region * (size_t)r; }
  flag_t* A(int owner, int src) const { return (flag_t*)(region(owner) + lay_.off_A + (size_t)src * kLine); }
  flag_t* B(int owner, int src) const { return (flag_t*)(region(owner) + lay_.off_B + (size_t)src * kLine); }
  flag_t* C(int owner, int src) const { return (flag_t*)(region(owner) + lay_.off_C + (size_t)src * kLine); }
  flag_t* meta(int owner, int par, int src) const {
    return (flag_t*)(region(owner) + lay_.off_meta + ((size_t)par * (size_t)lay_.p + (size_t)src) * kLine);
  }
  flag_t* sent(int owner, int src) const {
    return (flag_t*)(region(owner) + lay_.off_mctl + (size_t)(2 * src) * kLine);
  }
  flag_t* acked(int owner, int src) const {
    return (flag_t*)(region(owner) + lay_.off_mctl + (size_t)(2 * src + 1) * kLine);
  }
  /** Member rank + 1 of the first member whose operation failed; 0 while all is well. */
  flag_t* poison() const { return (flag_t*)(region(0) + lay_.off_poison); }
  char* stage(int r, int par) const { return region(r) + lay_.off_stage + (size_t)par * lay_.half; }
  char* mbox(int owner, int src, int slot) const {
    return region(owner) + lay_.off_mbox + ((size_t)src * 2 + (size_t)slot) * lay_.slot;
  }

 private:
  Layout lay_;
  std::string name_;
  size_t bytes_ = 0;
  char* base_ = nullptr;
};

}  // namespace host
}  // namespace internal

using namespace internal;
using namespace internal::host;

HostCommunicator::Impl::Impl(const Group& g)
    : p(g.size()), me(g.rank()), send_next((size_t)g.size()), send_serving((size_t)g.size()),
      recv_next((size_t)g.size()), recv_serving((size_t)g.size()), sent_count((size_t)g.size(), 0),
      acked_count((size_t)g.size(), 0) {
  world = g.world();
  world_rank_of = g.members();
  for (int i = 0; i < p; ++i) {
    send_next[(size_t)i] = 0; send_serving[(size_t)i] = 0;
    recv_next[(size_t)i] = 0; recv_serving[(size_t)i] = 0;
  }
  if (g.single_node()) {
    const uint64_t id = g.agree_on_id();
    ws.reset(new Workspace(g, id, tuning().host_stage_bytes, tuning().host_mailbox_bytes));
  } else {
    net.reset(new NetMesh(g));
    // Node structure of the members; a second level pays off when some node holds several of them.
    World* w = g.world();
    std::vector<std::string> names;
    node_of.resize((size_t)p);
    local_index.resize((size_t)p);
    std::vector<int> per_node;
    for (int r = 0; r < p; ++r) {
      const std::string& nm = w->node_of(g.world_rank_of(r));
      size_t k = 0;
      while (k < names.size() && names[k] != nm) ++k;
      if (k == names.size()) { names.push_back(nm); per_node.push_back(0); }
      node_of[(size_t)r] = (int)k;
      local_index[(size_t)r] = per_node[k]++;
    }
    const bool two_level = tuning().host_two_level && *std::max_element(per_node.begin(), per_node.end()) > 1 &&
                           names.size() > 1;
    if (two_level) {
      node_comm.reset(new HostCommunicator(g.split(node_of[(size_t)me], me)));
      const bool leader = local_index[(size_t)me] == 0;
      Group lg = g.split(leader ? 0 : 1, me);  // collective over all members; only the leaders build on it
      if (leader) leader_comm.reset(new HostCommunicator(lg));
      const bool even = *std::min_element(per_node.begin(), per_node.end()) == *std::max_element(per_node.begin(), per_node.end());
      if (even) rail_comm.reset(new HostCommunicator(g.split(local_index[(size_t)me], me)));
    }
  }
}

namespace {
/** (index of my node among the nodes of the group, my rank inside it, its population). */
void node_position(const Group& g, int* node, int* lrank, int* lsize) {
  *node = 0; *lrank = g.rank(); *lsize = g.size();
  World* w = g.world();
  if (!w || g.size() <= 1) return;
  const std::string& mine = w->node_of(g.world_rank_of(g.rank()));
  std::vector<std::string> seen;
  int before = 0, total = 0;
  for (int r = 0; r < g.size(); ++r) {
    const std::string& nm = w->node_of(g.world_rank_of(r));
    if (std::find(seen.begin(), seen.end(), nm) == seen.end()) seen.push_back(nm);
    if (nm == mine) { ++total; if (r < g.rank()) ++before; }
  }
  *node = (int)(std::find(seen.begin(), seen.end(), mine) - seen.begin());
  *lrank = before;
  *lsize = total;
}
}  // namespace

int HostCommunicator::local_rank() const { int n, r, s; node_position(group_, &n, &r, &s); return r; }
int HostCommunicator::local_size() const { int n, r, s; node_position(group_, &n, &r, &s); return s; }
HostCommunicator HostCommunicator::local() const {
  int n, r, s;
  node_position(group_, &n, &r, &s);
  return HostCommunicator(group_.split(n, group_.rank()));
}

void HostCommunicator::Impl::fail(const std::string& msg) {
  {
    std::lock_guard<std::mutex> g(fail_mu);
    if (failed.load()) return;
    fail_msg = msg;
    failed.store(true);
  }
  // First failure on this rank: let the peers know instead of leaving them to their time-outs.
  if (ws) {
    uint64_t none = 0;
    ws->poison()->compare_exchange_strong(none, (uint64_t)me + 1, std::memory_order_acq_rel);
  }
  if (net) net->shutdown_all();
  for (auto* sub : {node_comm.get(), leader_comm.get(), rail_comm.get()})
    if (sub) sub->abort("the communicator it serves failed: " + msg);
}

uint64_t HostCommunicator::Impl::poisoned_by() const {
  return ws ? ws->poison()->load(std::memory_order_acquire) : 0;
}

HostCommunicator::Impl::~Impl() {
  // Operations of this communicator were queued under its address; the slot can serve another one now.
  if (ProgressEngine* pe = get_progress_engine_if_any()) pe->release_key(this);
}

namespace {

inline uint64_t epoch(uint64_t seq, uint64_t sub) { return (seq << 24) | sub; }

inline size_t clamp_len(size_t count, size_t lo, size_t cap) {
  if (count <= lo) return 0;
  return std::min(cap, count - lo);
}

class CollState final : public HostState {
 public:
  CollState(HostCommunicator::Impl* ci, CollArgs&& a, Request req, uint64_t seq)
      : HostState(ci, std::move(req)), a_(std::move(a)), seq_(seq), ws_(*ci->ws), p_(ci->p), me_(ci->me) {
    esz_ = dtype_size(a_.dt);
    const Layout& L = ws_.lay();
    full_e_ = L.half / esz_;
    cap_b_ = (L.half / (size_t)p_) / kLine * kLine;
    cap_e_ = cap_b_ / esz_;
    if (cap_e_ == 0) throw_al_exception("host staging too small for ", p_, " ranks");
    if (!a_.vector) {
      // Synthesize uniform count tables so that one code path serves both forms.
      a_.send_counts.assign((size_t)p_, a_.count);
      a_.recv_counts.assign((size_t)p_, a_.count);
      a_.send_displs.resize((size_t)p_);
      a_.recv_displs.resize((size_t)p_);
      for (int r = 0; r < p_; ++r) a_.send_displs[(size_t)r] = a_.recv_displs[(size_t)r] = (size_t)r * a_.count;
    }
    local_chunks_ = compute_local_chunks();
  }
  const char* get_name() const override {
    static const char* n[] = {"HostAllreduce", "HostReduce", "HostReduceScatter", "HostAllgather",
                              "HostAlltoall", "HostBcast", "HostGather", "HostScatter", "HostBarrier"};
    return n[(int)a_.kind];
  }
  std::string get_desc() const override { return build_string("seq=", seq_, " count=", a_.count, " chunk=", c_); }

  PEAction step() override {
    if (failed_) { publish_outcome(); return PEAction::complete; }
    for (;;) {
      switch (phase_) {
        case Phase::gate:
          // Collectives of one communicator run strictly one after another.
          if (ci_->done_seq.load(std::memory_order_acquire) != seq_ - 1) {
            if (ci_->failed.load()) { fail("communicator failed earlier: " + ci_->fail_msg); return done(); }
            return PEAction::cont;
          }
          if (ci_->failed.load()) { fail("communicator failed earlier: " + ci_->fail_msg); return done(); }
          phase_ = Phase::publish;
          break;
        case Phase::publish: {
          if (!inject_fault()) return done();
          const int par = (int)((seq_ + c_) & 1);
          publish(c_, par);
          if (c_ == 0) {
            for (int r = 0; r < p_; ++r)
              ws_.meta(r, (int)(seq_ & 1), me_)->store(local_chunks_, std::memory_order_relaxed);
          }
          for (int r = 0; r < p_; ++r) ws_.A(r, me_)->store(epoch(seq_, c_ + 1), std::memory_order_release);
          phase_ = Phase::wait_a;
          break;
        }
        case Phase::wait_a: {
          if (!all_reached(&Workspace::A, epoch(seq_, c_ + 1))) {
            if (missing_peer_gone(&Workspace::A, epoch(seq_, c_ + 1)) || timed_out("peers to arrive")) return done();
            return PEAction::cont;
          }
          progress_made();
          if (c_ == 0) {
            global_chunks_ = 1;
            for (int r = 0; r < p_; ++r)
              global_chunks_ = std::max<uint64_t>(global_chunks_,
                                                  ws_.meta(me_, (int)(seq_ & 1), r)->load(std::memory_order_relaxed));
          }
          const int par = (int)((seq_ + c_) & 1);
          const bool two_phase = consume_a(c_, par);
          if (two_phase) {
            for (int r = 0; r < p_; ++r) ws_.B(r, me_)->store(epoch(seq_, c_ + 1), std::memory_order_release);
            phase_ = Phase::wait_b;
          } else {
            phase_ = Phase::next_chunk;
          }
          break;
        }
        case Phase::wait_b: {
          if (!all_reached(&Workspace::B, epoch(seq_, c_ + 1))) {
            if (missing_peer_gone(&Workspace::B, epoch(seq_, c_ + 1)) || timed_out("peers' reduced slices")) return done();
            return PEAction::cont;
          }
          progress_made();
          consume_b(c_, (int)((seq_ + c_) & 1));
          phase_ = Phase::next_chunk;
          break;
        }
        case Phase::next_chunk:
          ++c_;
          if (c_ < global_chunks_) { phase_ = Phase::publish; break; }
          if (global_chunks_ > 1) {
            // After a multi-chunk op the next op may start on either half:
            // make sure every peer is done reading both.
            for (int r = 0; r < p_; ++r) ws_.C(r, me_)->store(epoch(seq_, 1), std::memory_order_release);
            phase_ = Phase::wait_c;
            break;
          }
          return done();
        case Phase::wait_c:
          if (!all_reached(&Workspace::C, epoch(seq_, 1))) {
            if (missing_peer_gone(&Workspace::C, epoch(seq_, 1)) || timed_out("the closing barrier")) return done();
            return PEAction::cont;
          }
          return done();
      }
    }
  }

 private:
  enum class Phase { gate, publish, wait_a, wait_b, next_chunk, wait_c };

  /** Host-side fault injection (Tuning::fault_*).  Returns false when this rank drops out of the op. */
  bool inject_fault() {
    const Tuning& t = tuning();
    if (t.fault_jitter_us > 0) {
      static thread_local std::minstd_rand rng((unsigned)(me_ * 7919 + 17));
      std::this_thread::sleep_for(std::chrono::microseconds((long)(rng() % (unsigned long)t.fault_jitter_us)));
    }
    if (t.fault_kind == 0 || c_ != 0 || get_world()->rank() != t.fault_rank || (long)seq_ != t.fault_op) return true;
    if (t.fault_kind == 2) {
      std::this_thread::sleep_for(std::chrono::milliseconds(t.fault_delay_ms));
      return true;
    }
    fail(build_string(get_name(), ": injected fault, rank ", me_, " does not signal operation ", seq_));
    return false;
  }

  PEAction done() {
    // Even a failed op releases the gate so that later ops can observe the failure.
    ci_->done_seq.store(seq_, std::memory_order_release);
    publish_outcome();
    return PEAction::complete;
  }

  /** One of the ranks whose flag is still behind has exited: fail now (its flag can never come). */
  bool missing_peer_gone(flag_t* (Workspace::*which)(int, int) const, uint64_t e) {
    for (int r = 0; r < p_; ++r) {
      if (r == me_ || (ws_.*which)(me_, r)->load(std::memory_order_acquire) >= e) continue;
      if (!peer_gone(r)) return false;  // one check per call keeps the wait loop cheap
      if ((ws_.*which)(me_, r)->load(std::memory_order_acquire) >= e) return false;  // it signalled before it left
      fail(build_string(get_name(), ": rank ", r, " has exited (its control connection is closed)"));
      return true;
    }
    return false;
  }

  bool all_reached(flag_t* (Workspace::*which)(int, int) const, uint64_t e) {
    for (int r = 0; r < p_; ++r)
      if ((ws_.*which)(me_, r)->load(std::memory_order_acquire) < e) return false;
    return true;
  }

  uint64_t compute_local_chunks() const {
    size_t need = 0, unit = full_e_;
    auto mx = [](const std::vector<size_t>& v) { return v.empty() ? size_t{0} : *std::max_element(v.begin(), v.end()); };
    switch (a_.kind) {
      case Coll::allreduce: case Coll::reduce: case Coll::bcast: need = a_.count; unit = full_e_; break;
      case Coll::reduce_scatter: need = mx(a_.recv_counts); unit = cap_e_; break;
      case Coll::allgather: need = mx(a_.recv_counts); unit = full_e_; break;
      case Coll::alltoall: need = std::max(mx(a_.send_counts), mx(a_.recv_counts)); unit = cap_e_; break;
      case Coll::gather:
        need = me_ == a_.root ? mx(a_.recv_counts) : a_.send_counts[(size_t)me_];
        unit = full_e_;
        break;
      case Coll::scatter:
        need = me_ == a_.root ? mx(a_.send_counts) : a_.recv_counts[(size_t)me_];
        unit = cap_e_;
        break;
      case Coll::barrier: need = 0; break;
    }
    return std::max<uint64_t>(1, ceil_div(need, unit));
  }

  const char* sptr(size_t elem) const { return (const char*)a_.send + elem * esz_; }
  char* rptr(size_t elem) const { return (char*)a_.recv + elem * esz_; }

  void publish(uint64_t c, int par) {
    char* st = ws_.stage(me_, par);
    switch (a_.kind) {
      case Coll::allreduce: case Coll::reduce: {
        const size_t lo = c * full_e_, len = clamp_len(a_.count, lo, full_e_);
        if (len && a_.send) memcpy(st, sptr(lo), len * esz_);
        break;
      }
      case Coll::bcast: {
        if (me_ != a_.root) break;
        const size_t lo = c * full_e_, len = clamp_len(a_.count, lo, full_e_);
        if (len) memcpy(st, sptr(lo), len * esz_);
        break;
      }
      case Coll::allgather: case Coll::gather: {
        const size_t lo = c * full_e_, len = clamp_len(a_.send_counts[(size_t)me_], lo, full_e_);
        if (len && a_.send) memcpy(st, sptr(lo), len * esz_);
        break;
      }
      case Coll::reduce_scatter: case Coll::alltoall: case Coll::scatter: {
        if (a_.kind == Coll::scatter && me_ != a_.root) break;
        const size_t lo = c * cap_e_;
        for (int d = 0; d < p_; ++d) {
          const size_t cnt = a_.kind == Coll::reduce_scatter ? a_.recv_counts[(size_t)d] : a_.send_counts[(size_t)d];
          const size_t len = clamp_len(cnt, lo, cap_e_);
          if (len && a_.send) memcpy(st + (size_t)d * cap_b_, sptr(a_.send_displs[(size_t)d] + lo), len * esz_);
        }
        break;
      }
      case Coll::barrier: break;
    }
  }

  /** Work after the first handshake; returns true when a second (B) handshake follows. */
  bool consume_a(uint64_t c, int par) {
    switch (a_.kind) {
      case Coll::allreduce: {
        const size_t lo = c * full_e_, len = clamp_len(a_.count, lo, full_e_);
        std::vector<const void*> srcs((size_t)p_);
        if (len * esz_ <= 16384 || p_ == 1) {
          for (int r = 0; r < p_; ++r) srcs[(size_t)r] = ws_.stage(r, par);
          if (len) reduce_multi(a_.dt, a_.op, rptr(lo), srcs.data(), p_, len);
          return false;
        }
        const size_t per = ceil_div(len, (size_t)p_);
        const size_t s_lo = std::min(len, (size_t)me_ * per), s_len = clamp_len(len, s_lo, per);
        for (int r = 0; r < p_; ++r) srcs[(size_t)r] = ws_.stage(r, par) + s_lo * esz_;
        if (s_len) reduce_multi(a_.dt, a_.op, ws_.stage(me_, par) + s_lo * esz_, srcs.data(), p_, s_len);
        return true;
      }
      case Coll::reduce: {
        if (me_ != a_.root) return false;
        const size_t lo = c * full_e_, len = clamp_len(a_.count, lo, full_e_);
        std::vector<const void*> srcs((size_t)p_);
        for (int r = 0; r < p_; ++r) srcs[(size_t)r] = ws_.stage(r, par);
        if (len) reduce_multi(a_.dt, a_.op, rptr(lo), srcs.data(), p_, len);
        return false;
      }
      case Coll::reduce_scatter: {
        const size_t lo = c * cap_e_, len = clamp_len(a_.recv_counts[(size_t)me_], lo, cap_e_);
        std::vector<const void*> srcs((size_t)p_);
        for (int r = 0; r < p_; ++r) srcs[(size_t)r] = ws_.stage(r, par) + (size_t)me_ * cap_b_;
        if (len) reduce_multi(a_.dt, a_.op, rptr(lo), srcs.data(), p_, len);
        return false;
      }
      case Coll::allgather: {
        const size_t lo = c * full_e_;
        for (int r = 0; r < p_; ++r) {
          const size_t len = clamp_len(a_.recv_counts[(size_t)r], lo, full_e_);
          if (len) memcpy(rptr(a_.recv_displs[(size_t)r] + lo), ws_.stage(r, par), len * esz_);
        }
        return false;
      }
      case Coll::alltoall: {
        const size_t lo = c * cap_e_;
        for (int r = 0; r < p_; ++r) {
          const size_t len = clamp_len(a_.recv_counts[(size_t)r], lo, cap_e_);
          if (len) memcpy(rptr(a_.recv_displs[(size_t)r] + lo), ws_.stage(r, par) + (size_t)me_ * cap_b_, len * esz_);
        }
        return false;
      }
      case Coll::bcast: {
        if (me_ == a_.root) return false;
        const size_t lo = c * full_e_, len = clamp_len(a_.count, lo, full_e_);
        if (len) memcpy(rptr(lo), ws_.stage(a_.root, par), len * esz_);
        return false;
      }
      case Coll::gather: {
        if (me_ != a_.root) return false;
        const size_t lo = c * full_e_;
        for (int r = 0; r < p_; ++r) {
          const size_t len = clamp_len(a_.recv_counts[(size_t)r], lo, full_e_);
          if (len) memcpy(rptr(a_.recv_displs[(size_t)r] + lo), ws_.stage(r, par), len * esz_);
        }
        return false;
      }
      case Coll::scatter: {
        if (!a_.recv) return false;
        const size_t lo = c * cap_e_, len = clamp_len(a_.recv_counts[(size_t)me_], lo, cap_e_);
        if (len) memcpy(rptr(lo), ws_.stage(a_.root, par) + (size_t)me_ * cap_b_, len * esz_);
        return false;
      }
      case Coll::barrier: return false;
    }
    return false;
  }

  void consume_b(uint64_t c, int par) {
    // Only allreduce has a second phase: gather every owner's reduced slice.
    const size_t lo = c * full_e_, len = clamp_len(a_.count, lo, full_e_);
    const size_t per = ceil_div(len, (size_t)p_);
    for (int s = 0; s < p_; ++s) {
      const size_t s_lo = std::min(len, (size_t)s * per), s_len = clamp_len(len, s_lo, per);
      if (s_len) memcpy(rptr(lo + s_lo), ws_.stage(s, par) + s_lo * esz_, s_len * esz_);
    }
  }

  CollArgs a_;
  uint64_t seq_;
  Workspace& ws_;
  int p_, me_;
  size_t esz_ = 1, full_e_ = 0, cap_b_ = 0, cap_e_ = 0;
  uint64_t local_chunks_ = 1, global_chunks_ = 1, c_ = 0;
  Phase phase_ = Phase::gate;
};

/**
 * Point-to-point state: any number of sends and receives progressing together
 * (Send, Recv, SendRecv and MultiSendRecv are all instances).  Each ordered
 * pair has a two-slot mailbox in the receiver's region; `sent` is advanced by
 * the sender, `acked` by the receiver.  Transfers between the same pair are
 * served in call order through per-pair tickets.
 */
class P2PState final : public HostState {
 public:
  P2PState(HostCommunicator::Impl* ci, std::vector<P2PItem>&& items, Request req, const char* name)
      : HostState(ci, std::move(req)), ws_(*ci->ws), name_(name) {
    for (auto& it : items) {
      Xfer x;
      x.item = it;
      auto& next = it.is_send ? ci->send_next : ci->recv_next;
      x.ticket = next[(size_t)it.peer].fetch_add(1);
      x.pieces = std::max<size_t>(1, ceil_div(it.bytes, ws_.lay().slot));
      xfers_.push_back(x);
    }
  }
  const char* get_name() const override { return name_; }
  std::string get_desc() const override { return build_string("transfers=", xfers_.size()); }
  RunType get_run_type() const override { return RunType::unbounded; }

  PEAction step() override {
    if (failed_) { publish_outcome(); return PEAction::complete; }
    bool all_done = true, moved = false;
    const size_t slot = ws_.lay().slot;
    const int me = ci_->me;
    for (auto& x : xfers_) {
      if (x.done) continue;
      all_done = false;
      const int peer = x.item.peer;
      auto& serving = x.item.is_send ? ci_->send_serving : ci_->recv_serving;
      if (serving[(size_t)peer].load(std::memory_order_acquire) != x.ticket) continue;
      if (x.item.is_send) {
        uint64_t& sent = ci_->sent_count[(size_t)peer];
        while (x.piece < x.pieces) {
          const uint64_t acked = ws_.acked(peer, me)->load(std::memory_order_acquire);
          if (sent - acked >= 2) break;  // no free slot
          const size_t off = x.piece * slot, len = std::min(slot, x.item.bytes - std::min(x.item.bytes, off));
          if (len) memcpy(ws_.mbox(peer, me, (int)(sent & 1)), (const char*)x.item.sbuf + off, len);
          ++sent;
          ws_.sent(peer, me)->store(sent, std::memory_order_release);
          ++x.piece;
          moved = true;
        }
      } else {
        uint64_t& acked = ci_->acked_count[(size_t)peer];
        while (x.piece < x.pieces) {
          const uint64_t sent = ws_.sent(me, peer)->load(std::memory_order_acquire);
          if (sent == acked) break;  // nothing arrived yet
          const size_t off = x.piece * slot, len = std::min(slot, x.item.bytes - std::min(x.item.bytes, off));
          if (len) memcpy((char*)x.item.rbuf + off, ws_.mbox(me, peer, (int)(acked & 1)), len);
          ++acked;
          ws_.acked(me, peer)->store(acked, std::memory_order_release);
          ++x.piece;
          moved = true;
        }
      }
      if (x.piece == x.pieces) {
        x.done = true;
        serving[(size_t)peer].store(x.ticket + 1, std::memory_order_release);
      }
    }
    if (all_done) {
      publish_outcome();
      return PEAction::complete;
    }
    if (moved) progress_made();
    else if (pending_peer_gone() || timed_out("the matching send/receive")) {
      // Release the tickets so that later transfers fail fast instead of queueing forever.
      for (auto& x : xfers_)
        if (!x.done) {
          auto& serving = x.item.is_send ? ci_->send_serving : ci_->recv_serving;
          if (serving[(size_t)x.item.peer].load() == x.ticket) serving[(size_t)x.item.peer].store(x.ticket + 1);
        }
      publish_outcome();
      return PEAction::complete;
    }
    return PEAction::cont;
  }

 private:
  /** The peer of a transfer that is at the head of its queue has exited and left nothing to read. */
  bool pending_peer_gone() {
    const int me = ci_->me;
    for (auto& x : xfers_) {
      if (x.done) continue;
      const int peer = x.item.peer;
      auto& serving = x.item.is_send ? ci_->send_serving : ci_->recv_serving;
      if (peer == me || serving[(size_t)peer].load(std::memory_order_acquire) != x.ticket) continue;
      if (!peer_gone(peer)) return false;  // one check per call
      if (!x.item.is_send &&
          ws_.sent(me, peer)->load(std::memory_order_acquire) != ci_->acked_count[(size_t)peer])
        return false;  // it left, but its message is in the mailbox
      fail(build_string(name_, ": rank ", peer, " has exited (its control connection is closed)"));
      return true;
    }
    return false;
  }

  struct Xfer {
    P2PItem item;
    uint64_t ticket = 0;
    size_t pieces = 1, piece = 0;
    bool done = false;
  };
  Workspace& ws_;
  const char* name_;
  std::vector<Xfer> xfers_;
};

}  // namespace

namespace {
/** Block the caller until a request handed to the progress engine completes; rethrow its failure. */
void wait_for(const Request& r) {
  unsigned spins = 0;
  while (r->status.load(std::memory_order_acquire) == 0) {
    if (++spins < 200) AL_CPU_RELAX();
    else std::this_thread::yield();
  }
  if (r->status.load() == 2) throw_al_exception(r->error);
}
}  // namespace

namespace internal {
namespace host {
HostState* make_collective_state(HostCommunicator::Impl* ci, CollArgs&& args, Request req, uint64_t seq) {
  if (ci->node_comm) {
    if (HostState* st = make_hier_collective(ci, args, req, seq)) return st;  // leaves args alone when it declines
  }
  if (ci->net) return make_net_collective(ci, std::move(args), std::move(req), seq);
  return new CollState(ci, std::move(args), std::move(req), seq);
}
}  // namespace host
}  // namespace internal

HostCommunicator::HostCommunicator() : HostCommunicator(Group::world_group(get_world())) {}

HostCommunicator::HostCommunicator(const Group& group) : group_(group), impl_(new Impl(group)) {}

HostCommunicator::~HostCommunicator() = default;
HostCommunicator::HostCommunicator(HostCommunicator&&) noexcept = default;
HostCommunicator& HostCommunicator::operator=(HostCommunicator&&) noexcept = default;

void HostCommunicator::collective(CollArgs&& args, Request* req) {
  Impl* ci = impl_.get();
  if (ci->failed.load()) throw_al_exception("communicator is in a failed state: ", ci->fail_msg);
  if (args.root < 0 || args.root >= ci->p) throw_al_exception("root ", args.root, " out of range for ", ci->p, " rank(s)");
  if (args.kind == Coll::allreduce || args.kind == Coll::reduce || args.kind == Coll::reduce_scatter) {
    if (!reduction_supported(args.dt, args.op))
      throw_al_exception("reduction ", reduction_name(args.op), " is not defined for ", dtype_name(args.dt));
  }
  const uint64_t seq = ci->next_seq.fetch_add(1);
  ci->n_coll.fetch_add(1, std::memory_order_relaxed);
  {
    size_t elems = args.count;
    if (args.vector) { elems = 0; for (size_t c : args.send_counts) elems += c; }
    else if (args.kind == Coll::alltoall || args.kind == Coll::scatter || args.kind == Coll::reduce_scatter)
      elems *= (size_t)ci->p;
    if (args.send || args.kind == Coll::allreduce)
      ci->n_bytes.fetch_add(elems * dtype_size(args.dt), std::memory_order_relaxed);
  }
  Request r = std::make_shared<ReqState>();
  std::unique_ptr<HostState> st(make_collective_state(ci, std::move(args), r, seq));
  if (req) {
    *req = r;
    get_progress_engine()->enqueue(st.release());
  } else if (tuning().host_serialize) {
    // Every operation, blocking ones included, runs on the progress thread; the caller only waits.
    get_progress_engine()->enqueue(st.release());
    wait_for(r);
  } else {
    run_inline(*st);
    if (r->status.load() == 2) throw_al_exception(r->error);
  }
}

void HostCommunicator::p2p(std::vector<P2PItem>&& items, Request* req, const char* name) {
  Impl* ci = impl_.get();
  if (ci->failed.load()) throw_al_exception("communicator is in a failed state: ", ci->fail_msg);
  // A buffer that is both sent and received (in-place SendRecv) is sent from a
  // private copy so that arriving data cannot overtake the departing data.
  std::vector<void*> temps;
  for (auto& s : items) {
    if (!s.is_send || s.bytes == 0) continue;
    for (auto& r : items) {
      if (r.is_send || r.bytes == 0) continue;
      const char* sb = (const char*)s.sbuf;
      const char* rb = (const char*)r.rbuf;
      if (sb < rb + r.bytes && rb < sb + s.bytes) {
        void* t = mempool.allocate_bytes(MemoryType::HOST, s.bytes);
        memcpy(t, s.sbuf, s.bytes);
        s.sbuf = t;
        temps.push_back(t);
        break;
      }
    }
  }
  for (auto& it : items)
    if (it.peer < 0 || it.peer >= ci->p) throw_al_exception("point-to-point peer ", it.peer, " out of range");
  ci->n_p2p.fetch_add(1, std::memory_order_relaxed);
  for (auto& it : items)
    if (it.is_send) ci->n_bytes.fetch_add(it.bytes, std::memory_order_relaxed);
  Request r = std::make_shared<ReqState>();
  std::unique_ptr<HostState> st(ci->net ? make_net_p2p(ci, std::move(items), r, name)
                                        : new P2PState(ci, std::move(items), r, name));
  for (void* t : temps) st->adopt_temp(t);
  if (req) {
    *req = r;
    get_progress_engine()->enqueue(st.release());
  } else if (tuning().host_serialize) {
    // Every operation, blocking ones included, runs on the progress thread; the caller only waits.
    get_progress_engine()->enqueue(st.release());
    wait_for(r);
  } else {
    run_inline(*st);
    if (r->status.load() == 2) throw_al_exception(r->error);
  }
}

internal::host::CommStats HostCommunicator::stats() const {
  internal::host::CommStats s;
  s.collectives = impl_->n_coll.load();
  s.p2p_ops = impl_->n_p2p.load();
  s.bytes = impl_->n_bytes.load();
  s.failures = impl_->n_fail.load();
  return s;
}

void HostCommunicator::abort(const std::string& why) { impl_->fail(why); }

HostCommunicator HostCommunicator::from_ranks(const std::vector<int>& world_ranks) {
  return HostCommunicator(Group(get_world(), world_ranks));
}

bool HostCommunicator::failed() const { return impl_->failed.load(); }

}  // namespace Al
