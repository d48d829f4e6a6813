// Two-level collectives of a host communicator that spans nodes: shared memory
// inside each node, sockets between the nodes' first members.
//
// Small allreduce = reduce to the node's first member, allreduce among the first
// members, broadcast inside the node; bcast and barrier are composed the same
// way (the latency path, up to Tuning::host_two_level_max_bytes).  Large
// allreduce, when every node holds the same number of members = reduce-scatter
// inside the node, allreduce of each slice among the members with the same
// node-local rank (all of a node's members use their connections at once, and
// only 1/local_size of the vector crosses the network per member), allgather
// inside the node.  Everything else, and allreduce with the averaging
// operator, uses the flat socket path.  The parts are ordinary operations of the two
// sub-communicators, run one after another by one composite state, so the
// composite inherits their time-outs and failure reports.
#include <algorithm>
#include <memory>

#include "host_impl.hpp"

namespace Al {
namespace internal {
namespace host {

namespace {

class HierCollState final : public HostState {
 public:
  HierCollState(HostCommunicator::Impl* ci, const CollArgs& a, Request req, uint64_t seq)
      : HostState(ci, std::move(req)), kind_(a.kind), seq_(seq) {
    HostCommunicator::Impl* node = ci->node_comm->impl();
    HostCommunicator::Impl* lead = ci->leader_comm ? ci->leader_comm->impl() : nullptr;
    const bool leader = lead != nullptr;
    auto base = [&](Coll kind) {
      CollArgs s;
      s.kind = kind; s.dt = a.dt; s.op = a.op; s.count = a.count; s.root = 0;
      return s;
    };
    switch (a.kind) {
      case Coll::allreduce: {
        if (a.count * dtype_size(a.dt) > tuning().host_two_level_max_bytes) {
          // Bandwidth path over the rails.
          const int L = node->p, li = node->me;
          const size_t esz = dtype_size(a.dt);
          std::vector<size_t> counts((size_t)L), displs((size_t)L);
          const size_t per = (a.count + (size_t)L - 1) / (size_t)L;
          for (int r = 0; r < L; ++r) {
            displs[(size_t)r] = std::min(a.count, (size_t)r * per);
            counts[(size_t)r] = std::min(per, a.count - displs[(size_t)r]);
          }
          char* slice = (char*)a.recv + displs[(size_t)li] * esz;  // this member's slice, reduced in place in recv
          CollArgs rs = base(Coll::reduce_scatter);
          rs.vector = true;
          rs.send = a.send;
          rs.recv = slice;
          rs.recv_counts = counts; rs.send_counts = counts; rs.send_displs = displs;
          rs.recv_displs.assign((size_t)L, 0);
          add(node, std::move(rs));
          CollArgs ar = base(Coll::allreduce);
          ar.count = counts[(size_t)li];
          ar.send = slice; ar.recv = slice;
          add(ci->rail_comm->impl(), std::move(ar));
          CollArgs ag = base(Coll::allgather);
          ag.vector = true;
          ag.send = slice;
          ag.recv = a.recv;
          ag.recv_counts = counts; ag.recv_displs = displs; ag.send_counts = counts;
          ag.send_displs.assign((size_t)L, 0);
          add(node, std::move(ag));
          break;
        }
        CollArgs r = base(Coll::reduce);
        r.send = a.send;
        r.recv = leader ? a.recv : nullptr;
        add(node, std::move(r));
        if (leader) {
          CollArgs ar = base(Coll::allreduce);
          ar.send = a.recv; ar.recv = a.recv;
          add(lead, std::move(ar));
        }
        CollArgs b = base(Coll::bcast);
        b.send = a.recv; b.recv = a.recv;
        add(node, std::move(b));
        break;
      }
      case Coll::bcast: {
        const int root_node = ci->node_of[(size_t)a.root];
        const bool on_root_node = ci->node_of[(size_t)ci->me] == root_node;
        CollArgs b = base(Coll::bcast);
        b.send = a.recv; b.recv = a.recv;
        if (on_root_node) {
          CollArgs first = b;
          first.root = ci->local_index[(size_t)a.root];
          add(node, std::move(first));
        }
        if (leader) {
          CollArgs mid = b;
          mid.root = root_node;  // the leaders' ranks are the node indices
          add(lead, std::move(mid));
        }
        if (!on_root_node) add(node, std::move(b));
        break;
      }
      case Coll::barrier: {
        add(node, base(Coll::barrier));
        if (leader) add(lead, base(Coll::barrier));
        add(node, base(Coll::barrier));
        break;
      }
      default: break;
    }
  }
  const char* get_name() const override {
    return kind_ == Coll::allreduce ? "HierAllreduce" : kind_ == Coll::bcast ? "HierBcast" : "HierBarrier";
  }
  std::string get_desc() const override { return build_string("seq=", seq_, " part=", cur_, "/", parts_.size()); }

  PEAction step() override {
    if (failed_) return finish();
    if (!my_turn_) {
      const bool turn = ci_->done_seq.load(std::memory_order_acquire) == seq_ - 1;
      if (ci_->failed.load()) { fail("communicator failed earlier: " + ci_->fail_msg); return finish(); }
      if (!turn) return PEAction::cont;
      my_turn_ = true;
    }
    while (cur_ < parts_.size()) {
      Part& p = parts_[cur_];
      if (!p.started) { p.st->start(); p.started = true; }
      if (p.st->step() != PEAction::complete) {
        if (ci_->failed.load(std::memory_order_acquire)) {  // aborted by the caller
          fail("communicator failed: " + ci_->fail_msg);
          return finish();
        }
        return PEAction::cont;
      }
      if (p.req->status.load(std::memory_order_acquire) == 2) { fail(p.req->error); return finish(); }
      ++cur_;
    }
    return finish();
  }

 private:
  struct Part {
    std::unique_ptr<HostState> st;
    Request req;
    bool started = false;
  };
  void add(HostCommunicator::Impl* sub, CollArgs&& args) {
    Part p;
    p.req = std::make_shared<ReqState>();
    // Sequence numbers of the sub-communicators are taken now, at call time, in the same order on every member.
    const uint64_t seq = sub->next_seq.fetch_add(1);
    p.st.reset(make_collective_state(sub, std::move(args), p.req, seq));
    parts_.push_back(std::move(p));
  }
  PEAction finish() {
    ci_->done_seq.store(seq_, std::memory_order_release);
    publish_outcome();
    return PEAction::complete;
  }

  Coll kind_;
  uint64_t seq_;
  bool my_turn_ = false;
  std::vector<Part> parts_;
  size_t cur_ = 0;
};

}  // namespace

HostState* make_hier_collective(HostCommunicator::Impl* ci, CollArgs& args, Request req, uint64_t seq) {
  const bool fits = args.kind == Coll::bcast || args.kind == Coll::barrier ||
                    (args.kind == Coll::allreduce && args.op != ReductionOperator::avg);
  if (!fits || !ci->node_comm) return nullptr;
  // Large messages are bandwidth-bound: the flat path moves them over every member's connections at
  // once, the two-level path over one connection per node.  (Every member evaluates the same test.)
  const bool large = args.count * dtype_size(args.dt) > tuning().host_two_level_max_bytes;
  if (large && !(args.kind == Coll::allreduce && ci->rail_comm)) return nullptr;
  return new HierCollState(ci, args, std::move(req), seq);
}

}  // namespace host
}  // namespace internal
}  // namespace Al
