// Socket data plane of host communicators that span nodes (see host_net.hpp):
// connection mesh, non-blocking message rounds, and the collective and
// point-to-point state machines built on them.
#include "host_net.hpp"

#include <errno.h>
#include <fcntl.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <deque>
#include <functional>

#include "al/host/reduce.hpp"
#include "al/progress.hpp"
#include "al/runtime.hpp"
#include "al/util/meta.hpp"
#include "host_impl.hpp"

namespace Al {
namespace internal {
namespace host {

namespace {

constexpr uint32_t kMagic = 0x414c4e54u;  // "ALNT"
constexpr size_t kMaxBurst = size_t{4} << 20;  // bytes moved per message per progress call

struct MeshHello { int32_t rank; int32_t channel; };

void blocking_write(int fd, const void* buf, size_t n) {
  const char* p = (const char*)buf;
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      throw_al_exception("communicator setup: send failed: ", strerror(errno));
    }
    p += w;
    n -= (size_t)w;
  }
}

void blocking_read(int fd, void* buf, size_t n, double deadline) {
  char* p = (char*)buf;
  while (n) {
    pollfd pf{fd, POLLIN, 0};
    if (get_time() > deadline) throw_al_exception("communicator setup: timed out reading a peer's greeting");
    if (::poll(&pf, 1, 200) <= 0) continue;
    ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) throw_al_exception("communicator setup: a peer closed the connection");
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      throw_al_exception("communicator setup: recv failed: ", strerror(errno));
    }
    p += r;
    n -= (size_t)r;
  }
}

void make_data_socket(int fd) {
  const int flags = ::fcntl(fd, F_GETFL, 0);
  ::fcntl(fd, F_SETFL, flags | O_NONBLOCK);
  int one = 1;
  ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));  // small messages must not wait for Nagle's timer
  int buf = 4 << 20;
  ::setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &buf, sizeof(buf));
  ::setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &buf, sizeof(buf));
}

}  // namespace

NetMesh::NetMesh(const Group& g) : p_(g.size()), me_(g.rank()) {
  fds_[0].assign((size_t)p_, -1);
  fds_[1].assign((size_t)p_, -1);
  const double tmo = env_double("AL_BOOTSTRAP_TIMEOUT_S", 120.0);
  int port = 0;
  const int lfd = bootstrap_tcp_listen(&port);
  try {
    std::vector<int32_t> ports((size_t)p_);
    int32_t mine = port;
    g.allgather(&mine, ports.data(), sizeof(int32_t));  // everyone listens before anyone connects
    // The higher rank of a pair opens both connections.
    for (int peer = 0; peer < me_; ++peer) {
      const std::string& ip = g.world()->address_of(g.world_rank_of(peer));
      for (int ch = 0; ch < 2; ++ch) {
        const int fd = bootstrap_tcp_connect(ip, ports[(size_t)peer], tmo);
        if (fd < 0) throw_al_exception("communicator setup: rank ", me_, " could not connect to rank ", peer, " at ", ip, ":", ports[(size_t)peer]);
        fds_[ch][(size_t)peer] = fd;
        MeshHello h{me_, ch};
        blocking_write(fd, &h, sizeof(h));
      }
    }
    const double deadline = get_time() + tmo;
    for (int left = 2 * (p_ - 1 - me_); left > 0; --left) {
      int fd = -1;
      for (;;) {
        pollfd pf{lfd, POLLIN, 0};
        if (::poll(&pf, 1, 200) > 0) {
          fd = ::accept4(lfd, nullptr, nullptr, SOCK_CLOEXEC);
          if (fd >= 0) break;
          if (errno != EINTR && errno != EAGAIN) throw_al_exception("communicator setup: accept(): ", strerror(errno));
        }
        if (get_time() > deadline)
          throw_al_exception("communicator setup: rank ", me_, " timed out waiting for ", left, " connection(s)");
      }
      MeshHello h{-1, -1};
      try {
        blocking_read(fd, &h, sizeof(h), deadline);
      } catch (...) {
        ::close(fd);
        throw;
      }
      if (h.rank <= me_ || h.rank >= p_ || h.channel < 0 || h.channel > 1 || fds_[h.channel][(size_t)h.rank] != -1) {
        ::close(fd);
        throw_al_exception("communicator setup: unexpected connection (rank ", h.rank, ", channel ", h.channel, ")");
      }
      fds_[h.channel][(size_t)h.rank] = fd;
    }
  } catch (...) {
    ::close(lfd);
    for (auto& v : fds_)
      for (int fd : v)
        if (fd >= 0) ::close(fd);
    throw;
  }
  ::close(lfd);
  for (auto& v : fds_)
    for (int fd : v)
      if (fd >= 0) make_data_socket(fd);
}

void NetMesh::shutdown_all() const {
  for (const auto& ch : fds_)
    for (int fd : ch)
      if (fd >= 0) ::shutdown(fd, SHUT_RDWR);
}

NetMesh::~NetMesh() {
  for (auto& v : fds_)
    for (int fd : v)
      if (fd >= 0) ::close(fd);
}

// ---------------------------------------------------------------------------
// rounds
// ---------------------------------------------------------------------------
void NetRound::send(int peer, const void* buf, size_t bytes) {
  NetXfer x;
  x.peer = peer; x.is_send = true; x.buf = (char*)const_cast<void*>(buf); x.bytes = bytes;
  xfers_.push_back(x);
}

void NetRound::recv(int peer, void* buf, size_t bytes) {
  NetXfer x;
  x.peer = peer; x.is_send = false; x.buf = (char*)buf; x.bytes = bytes;
  xfers_.push_back(x);
}

void NetRound::seal(uint64_t seq, uint32_t round) {
  for (auto& x : xfers_) {
    x.hdr.magic = kMagic;
    x.hdr.round = round;
    x.hdr.seq = seq;
    x.hdr.bytes = x.bytes;
  }
}

int NetRound::waiting_for() const {
  for (auto& x : xfers_)
    if (!x.complete()) return x.peer;
  return -1;
}

NetRound::Status NetRound::progress(const NetMesh& mesh, int channel, bool* moved, std::string* err) {
  bool all = true;
  // busy[2*r + dir]: an earlier, incomplete message to (dir 0) / from (dir 1) rank r exists in this round.
  busy_.assign((size_t)mesh.size() * 2, 0);
  for (auto& x : xfers_) {
    if (x.complete()) continue;
    all = false;
    char& busy = busy_[(size_t)x.peer * 2 + (x.is_send ? 0 : 1)];
    if (busy) continue;
    busy = 1;
    const int fd = mesh.fd(channel, x.peer);
    for (;;) {
      const bool in_hdr = x.hdr_done < sizeof(NetHeader);
      char* p = in_hdr ? (char*)(x.is_send ? &x.hdr : &x.got) + x.hdr_done : x.buf + x.done;
      size_t left = in_hdr ? sizeof(NetHeader) - x.hdr_done : x.bytes - x.done;
      if (left == 0) break;
      left = std::min(left, kMaxBurst);
      ssize_t n;
      if (x.is_send && in_hdr && x.bytes) {
        // Header and the start of the payload leave in one segment.
        iovec iov[2] = {{p, left}, {x.buf, std::min(x.bytes, kMaxBurst)}};
        msghdr mh{};
        mh.msg_iov = iov;
        mh.msg_iovlen = 2;
        n = ::sendmsg(fd, &mh, MSG_DONTWAIT | MSG_NOSIGNAL);
        if (n > (ssize_t)left) {
          x.hdr_done = sizeof(NetHeader);
          x.done = (size_t)n - left;
          *moved = true;
          if (x.done < x.bytes) break;
          continue;
        }
      } else {
        n = x.is_send ? ::send(fd, p, left, MSG_DONTWAIT | MSG_NOSIGNAL) : ::recv(fd, p, left, MSG_DONTWAIT);
      }
      if (n > 0) {
        *moved = true;
        if (in_hdr) {
          x.hdr_done += (size_t)n;
          if (!x.is_send && x.hdr_done == sizeof(NetHeader) &&
              (x.got.magic != kMagic || x.got.seq != x.hdr.seq || x.got.round != x.hdr.round || x.got.bytes != x.hdr.bytes)) {
            *err = build_string("rank ", x.peer, " sent a message of ", x.got.bytes, " bytes (operation ", x.got.seq,
                                ", step ", x.got.round, ") where ", x.hdr.bytes, " bytes (operation ", x.hdr.seq, ", step ",
                                x.hdr.round, ") were expected: the ranks' calls do not match");
            return error;
          }
        } else {
          x.done += (size_t)n;
        }
        if ((size_t)n < left) break;             // the socket took / had less than asked: come back later
        if (!in_hdr && x.done < x.bytes) break;  // one burst per call keeps all peers moving together
        continue;
      }
      if (n == 0 && !x.is_send) {
        *err = build_string("rank ", x.peer, " closed the connection");
        return error;
      }
      if (errno == EINTR) continue;
      if (errno == EAGAIN || errno == EWOULDBLOCK) break;
      *err = build_string(x.is_send ? "send to rank " : "receive from rank ", x.peer, " failed: ", strerror(errno));
      return error;
    }
  }
  return all ? done : pending;
}

// ---------------------------------------------------------------------------
// collectives
// ---------------------------------------------------------------------------
namespace {

bool ranges_overlap(const void* a, size_t na, const void* b, size_t nb) {
  const char* x = (const char*)a;
  const char* y = (const char*)b;
  return na && nb && x < y + nb && y < x + na;
}

/**
 * A collective as a short list of rounds with local work after each.
 *
 * Algorithms (p ranks, direct connections between all pairs):
 *   allgather, gather, scatter, alltoall: one round of direct transfers
 *   reduce_scatter: every rank receives the p-1 other contributions to its
 *     slice and folds all p in rank order
 *   allreduce: reduce_scatter over balanced slices, then allgather of the
 *     reduced slices (small vectors: exchange everything, fold locally)
 *   reduce: like allreduce's first round, then the slices travel to the root
 *   bcast: root sends to everyone (large: scatter, then allgather)
 *   barrier: dissemination, ceil(log2 p) rounds of one byte
 * Folding in rank order by one owner per slice gives every rank bit-identical
 * results, as on the shared-memory path.
 */
class NetCollState final : public HostState {
 public:
  NetCollState(HostCommunicator::Impl* ci, CollArgs&& a, Request req, uint64_t seq)
      : HostState(ci, std::move(req)), a_(std::move(a)), seq_(seq), mesh_(*ci->net), p_(ci->p), me_(ci->me) {
    esz_ = dtype_size(a_.dt);
    if (!a_.vector) {
      a_.send_counts.assign((size_t)p_, a_.count);
      a_.recv_counts.assign((size_t)p_, a_.count);
      a_.send_displs.resize((size_t)p_);
      a_.recv_displs.resize((size_t)p_);
      for (int r = 0; r < p_; ++r) a_.send_displs[(size_t)r] = a_.recv_displs[(size_t)r] = (size_t)r * a_.count;
    }
  }
  const char* get_name() const override {
    static const char* n[] = {"NetAllreduce", "NetReduce", "NetReduceScatter", "NetAllgather",
                              "NetAlltoall", "NetBcast", "NetGather", "NetScatter", "NetBarrier"};
    return n[(int)a_.kind];
  }
  std::string get_desc() const override {
    return build_string("seq=", seq_, " count=", a_.count, " step=", cur_, "/", steps_.size());
  }

  PEAction step() override {
    if (failed_) return finish();
    if (!planned_) {
      // Collectives of one communicator run strictly one after another: they share the sockets.
      const bool my_turn = ci_->done_seq.load(std::memory_order_acquire) == seq_ - 1;
      if (ci_->failed.load()) { fail("communicator failed earlier: " + ci_->fail_msg); return finish(); }
      if (!my_turn) return PEAction::cont;
      plan();
      for (size_t i = 0; i < steps_.size(); ++i) steps_[i].round.seal(seq_, (uint32_t)i);
      planned_ = true;
    }
    while (cur_ < steps_.size()) {
      Step& s = steps_[cur_];
      bool moved = false;
      std::string err;
      const NetRound::Status st = s.round.progress(mesh_, kNetCollectives, &moved, &err);
      if (st == NetRound::error) { fail(build_string(get_name(), ": ", err)); return finish(); }
      if (st == NetRound::pending) {
        if (moved) progress_made();
        else {
          what_ = build_string("rank ", s.round.waiting_for());
          if (timed_out(what_.c_str())) return finish();
        }
        return PEAction::cont;
      }
      progress_made();
      if (s.after) s.after();
      ++cur_;
    }
    return finish();
  }

 private:
  struct Step {
    NetRound round;
    std::function<void()> after;
  };

  PEAction finish() {
    // Even a failed operation opens the gate so that later ones can observe the failure.
    ci_->done_seq.store(seq_, std::memory_order_release);
    publish_outcome();
    return PEAction::complete;
  }

  const char* S(size_t elem) const { return (const char*)a_.send + elem * esz_; }
  char* R(size_t elem) const { return (char*)a_.recv + elem * esz_; }
  Step& add_step() { steps_.emplace_back(); return steps_.back(); }

  /** Balanced slices of a vector of n elements: slice r = [lo(r), lo(r) + len(r)). */
  struct Slices {
    size_t n, per;
    size_t lo(int r) const { return std::min(n, (size_t)r * per); }
    size_t len(int r) const { return std::min(per, n - lo(r)); }
  };
  Slices slices(size_t n) const { return Slices{n, ceil_div(std::max<size_t>(n, 1), (size_t)p_)}; }

  /** Fold own contribution and the p-1 received ones (tmp[r], r != me) into out, in rank order. */
  void fold(void* out, const void* own, const std::vector<char*>& tmp, size_t n) {
    if (!n) return;
    std::vector<const void*> srcs((size_t)p_);
    for (int r = 0; r < p_; ++r) srcs[(size_t)r] = r == me_ ? own : (const void*)tmp[(size_t)r];
    reduce_multi(a_.dt, a_.op, out, srcs.data(), p_, n);
  }

  /** One temporary of `bytes` per peer (nullptr for this rank). */
  std::vector<char*> peer_temps(size_t bytes) {
    std::vector<char*> t((size_t)p_, nullptr);
    char* base = (char*)temp(bytes * (size_t)std::max(1, p_ - 1));
    int k = 0;
    for (int r = 0; r < p_; ++r)
      if (r != me_) t[(size_t)r] = base + (size_t)(k++) * bytes;
    return t;
  }

  void plan() {
    switch (a_.kind) {
      case Coll::barrier: {
        for (int k = 1; k < p_; k <<= 1) {
          Step& s = add_step();
          s.round.send((me_ + k) % p_, &token_, 1);
          s.round.recv((me_ - k + p_) % p_, &sink_, 1);
        }
        break;
      }
      case Coll::bcast: {
        const size_t n = a_.count, bytes = n * esz_;
        if (p_ <= 2 || bytes < (size_t{256} << 10)) {
          Step& s = add_step();
          if (me_ == a_.root) {
            for (int r = 0; r < p_; ++r)
              if (r != me_) s.round.send(r, S(0), bytes);
          } else {
            s.round.recv(a_.root, R(0), bytes);
          }
          break;
        }
        const Slices sl = slices(n);
        Step& s1 = add_step();  // scatter
        if (me_ == a_.root) {
          for (int r = 0; r < p_; ++r)
            if (r != me_) s1.round.send(r, S(sl.lo(r)), sl.len(r) * esz_);
        } else {
          s1.round.recv(a_.root, R(sl.lo(me_)), sl.len(me_) * esz_);
        }
        Step& s2 = add_step();  // allgather among the non-roots, root supplies its own slice
        for (int r = 0; r < p_; ++r) {
          if (r == me_) continue;
          if (r != a_.root) s2.round.send(r, me_ == a_.root ? S(sl.lo(me_)) : R(sl.lo(me_)), sl.len(me_) * esz_);
          if (me_ != a_.root) s2.round.recv(r, R(sl.lo(r)), sl.len(r) * esz_);
        }
        break;
      }
      case Coll::allgather: {
        char* own_dst = R(a_.recv_displs[(size_t)me_]);
        const size_t own_bytes = a_.recv_counts[(size_t)me_] * esz_;
        const char* src = a_.send ? S(0) : own_dst;
        if (src != own_dst && own_bytes) memmove(own_dst, src, own_bytes);
        Step& s = add_step();
        for (int r = 0; r < p_; ++r) {
          if (r == me_) continue;
          s.round.send(r, own_dst, own_bytes);
          s.round.recv(r, R(a_.recv_displs[(size_t)r]), a_.recv_counts[(size_t)r] * esz_);
        }
        break;
      }
      case Coll::gather: {
        Step& s = add_step();
        if (me_ == a_.root) {
          char* own_dst = R(a_.recv_displs[(size_t)me_]);
          const size_t own_bytes = a_.recv_counts[(size_t)me_] * esz_;
          if (a_.send && S(0) != own_dst && own_bytes) memmove(own_dst, S(0), own_bytes);
          for (int r = 0; r < p_; ++r)
            if (r != me_) s.round.recv(r, R(a_.recv_displs[(size_t)r]), a_.recv_counts[(size_t)r] * esz_);
        } else {
          s.round.send(a_.root, S(0), a_.send_counts[(size_t)me_] * esz_);
        }
        break;
      }
      case Coll::scatter: {
        Step& s = add_step();
        if (me_ == a_.root) {
          for (int r = 0; r < p_; ++r)
            if (r != me_) s.round.send(r, S(a_.send_displs[(size_t)r]), a_.send_counts[(size_t)r] * esz_);
          const size_t own_bytes = a_.send_counts[(size_t)me_] * esz_;
          if (a_.recv && R(0) != S(a_.send_displs[(size_t)me_]) && own_bytes)
            memmove(R(0), S(a_.send_displs[(size_t)me_]), own_bytes);
        } else {
          s.round.recv(a_.root, R(0), a_.recv_counts[(size_t)me_] * esz_);
        }
        break;
      }
      case Coll::alltoall: {
        Step& s = add_step();
        const bool in_place = (const void*)a_.send == (const void*)a_.recv;
        if (!in_place) {
          const size_t own = std::min(a_.send_counts[(size_t)me_], a_.recv_counts[(size_t)me_]) * esz_;
          if (own) memmove(R(a_.recv_displs[(size_t)me_]), S(a_.send_displs[(size_t)me_]), own);
          for (int r = 0; r < p_; ++r) {
            if (r == me_) continue;
            s.round.send(r, S(a_.send_displs[(size_t)r]), a_.send_counts[(size_t)r] * esz_);
            s.round.recv(r, R(a_.recv_displs[(size_t)r]), a_.recv_counts[(size_t)r] * esz_);
          }
          break;
        }
        // In place: what arrives would overwrite what has not left yet, so it lands in temporaries first.
        std::vector<char*> tmp((size_t)p_, nullptr);
        for (int r = 0; r < p_; ++r) {
          if (r == me_) continue;
          tmp[(size_t)r] = (char*)temp(a_.recv_counts[(size_t)r] * esz_);
          s.round.send(r, S(a_.send_displs[(size_t)r]), a_.send_counts[(size_t)r] * esz_);
          s.round.recv(r, tmp[(size_t)r], a_.recv_counts[(size_t)r] * esz_);
        }
        s.after = [this, tmp] {
          for (int r = 0; r < p_; ++r)
            if (r != me_ && a_.recv_counts[(size_t)r])
              memcpy(R(a_.recv_displs[(size_t)r]), tmp[(size_t)r], a_.recv_counts[(size_t)r] * esz_);
        };
        break;
      }
      case Coll::reduce_scatter: {
        const size_t cnt = a_.recv_counts[(size_t)me_];
        std::vector<char*> tmp = peer_temps(cnt * esz_);
        Step& s = add_step();
        for (int r = 0; r < p_; ++r) {
          if (r == me_) continue;
          s.round.send(r, S(a_.send_displs[(size_t)r]), a_.recv_counts[(size_t)r] * esz_);
          s.round.recv(r, tmp[(size_t)r], cnt * esz_);
        }
        s.after = [this, tmp, cnt] {
          const char* own = S(a_.send_displs[(size_t)me_]);
          if (own != R(0) && ranges_overlap(own, cnt * esz_, R(0), cnt * esz_)) {
            // In place with uneven counts the result can partly cover this rank's own slice.
            char* copy = (char*)temp(cnt * esz_);
            memcpy(copy, own, cnt * esz_);
            own = copy;
          }
          fold(R(0), own, tmp, cnt);
        };
        break;
      }
      case Coll::allreduce: {
        const size_t n = a_.count, bytes = n * esz_;
        if (bytes <= (size_t{16} << 10) || n < (size_t)p_) {
          std::vector<char*> tmp = peer_temps(bytes);
          Step& s = add_step();
          for (int r = 0; r < p_; ++r) {
            if (r == me_) continue;
            s.round.send(r, S(0), bytes);
            s.round.recv(r, tmp[(size_t)r], bytes);
          }
          s.after = [this, tmp, n] { fold(R(0), S(0), tmp, n); };
          break;
        }
        const Slices sl = slices(n);
        std::vector<char*> tmp = peer_temps(sl.len(me_) * esz_);
        Step& s1 = add_step();
        for (int r = 0; r < p_; ++r) {
          if (r == me_) continue;
          s1.round.send(r, S(sl.lo(r)), sl.len(r) * esz_);
          s1.round.recv(r, tmp[(size_t)r], sl.len(me_) * esz_);
        }
        s1.after = [this, tmp, sl] { fold(R(sl.lo(me_)), S(sl.lo(me_)), tmp, sl.len(me_)); };
        Step& s2 = add_step();
        for (int r = 0; r < p_; ++r) {
          if (r == me_) continue;
          s2.round.send(r, R(sl.lo(me_)), sl.len(me_) * esz_);
          s2.round.recv(r, R(sl.lo(r)), sl.len(r) * esz_);
        }
        break;
      }
      case Coll::reduce: {
        const size_t n = a_.count, bytes = n * esz_;
        if (p_ == 2 || bytes <= (size_t{64} << 10) || n < (size_t)p_) {
          Step& s = add_step();
          if (me_ == a_.root) {
            std::vector<char*> tmp = peer_temps(bytes);
            for (int r = 0; r < p_; ++r)
              if (r != me_) s.round.recv(r, tmp[(size_t)r], bytes);
            s.after = [this, tmp, n] { fold(R(0), S(0), tmp, n); };
          } else {
            s.round.send(a_.root, S(0), bytes);
          }
          break;
        }
        const Slices sl = slices(n);
        std::vector<char*> tmp = peer_temps(sl.len(me_) * esz_);
        char* reduced = me_ == a_.root ? R(sl.lo(me_)) : (char*)temp(sl.len(me_) * esz_);
        Step& s1 = add_step();
        for (int r = 0; r < p_; ++r) {
          if (r == me_) continue;
          s1.round.send(r, S(sl.lo(r)), sl.len(r) * esz_);
          s1.round.recv(r, tmp[(size_t)r], sl.len(me_) * esz_);
        }
        s1.after = [this, tmp, sl, reduced] { fold(reduced, S(sl.lo(me_)), tmp, sl.len(me_)); };
        Step& s2 = add_step();
        if (me_ == a_.root) {
          for (int r = 0; r < p_; ++r)
            if (r != me_) s2.round.recv(r, R(sl.lo(r)), sl.len(r) * esz_);
        } else {
          s2.round.send(a_.root, reduced, sl.len(me_) * esz_);
        }
        break;
      }
    }
  }

  CollArgs a_;
  uint64_t seq_;
  const NetMesh& mesh_;
  int p_, me_;
  size_t esz_ = 1;
  bool planned_ = false;
  std::deque<Step> steps_;  // references handed out by add_step() stay valid
  size_t cur_ = 0;
  std::string what_;
  char token_ = 1, sink_ = 0;
};

// ---------------------------------------------------------------------------
// point-to-point
// ---------------------------------------------------------------------------
/**
 * Sends and receives over the pair's point-to-point connection.  Transfers of
 * one direction of one pair run in call order (tickets), so the byte stream
 * needs no tags; the header carries the ticket and the size, and a receive
 * that meets a different size fails instead of misreading the stream.
 */
class NetP2PState final : public HostState {
 public:
  NetP2PState(HostCommunicator::Impl* ci, std::vector<P2PItem>&& items, Request req, const char* name)
      : HostState(ci, std::move(req)), mesh_(*ci->net), name_(name) {
    // Transfers to this rank itself are paired in order within the call and become copies.
    std::vector<P2PItem*> self_send, self_recv;
    for (auto& it : items) {
      if (it.peer != ci->me) continue;
      (it.is_send ? self_send : self_recv).push_back(&it);
    }
    if (self_send.size() != self_recv.size())
      self_error_ = "a transfer to this rank itself needs its counterpart in the same call (use SendRecv)";
    for (size_t k = 0; k < std::min(self_send.size(), self_recv.size()); ++k) {
      if (self_send[k]->bytes != self_recv[k]->bytes) { self_error_ = "send and receive sizes of a self transfer differ"; break; }
      if (self_send[k]->bytes) memmove(self_recv[k]->rbuf, self_send[k]->sbuf, self_send[k]->bytes);
    }
    for (auto& it : items) {
      if (it.peer == ci->me) continue;
      Xfer x;
      x.item = it;
      auto& next = it.is_send ? ci->send_next : ci->recv_next;
      x.ticket = next[(size_t)it.peer].fetch_add(1);
      xfers_.push_back(std::move(x));
    }
  }
  const char* get_name() const override { return name_; }
  std::string get_desc() const override { return build_string("transfers=", xfers_.size()); }
  RunType get_run_type() const override { return RunType::unbounded; }

  PEAction step() override {
    if (failed_) return finish();
    if (!self_error_.empty()) { fail(build_string(name_, ": ", self_error_)); return finish(); }
    bool all_done = true, moved = false;
    for (auto& x : xfers_) {
      if (x.done) continue;
      all_done = false;
      const int peer = x.item.peer;
      auto& serving = x.item.is_send ? ci_->send_serving : ci_->recv_serving;
      if (serving[(size_t)peer].load(std::memory_order_acquire) != x.ticket) continue;
      if (!x.started) {
        if (x.item.is_send) x.round.send(peer, x.item.sbuf, x.item.bytes);
        else x.round.recv(peer, x.item.rbuf, x.item.bytes);
        x.round.seal(x.ticket, 0);
        x.started = true;
      }
      std::string err;
      const NetRound::Status st = x.round.progress(mesh_, kNetPointToPoint, &moved, &err);
      if (st == NetRound::error) { fail(build_string(name_, ": ", err)); return finish(); }
      if (st == NetRound::done) {
        x.done = true;
        moved = true;
        serving[(size_t)peer].store(x.ticket + 1, std::memory_order_release);
      }
    }
    if (all_done) return finish();
    if (moved) progress_made();
    else if (timed_out("the matching send/receive")) return finish();
    return PEAction::cont;
  }

 private:
  struct Xfer {
    P2PItem item;
    uint64_t ticket = 0;
    NetRound round;
    bool started = false, done = false;
  };

  PEAction finish() {
    if (failed_) {
      // Pass the tickets on so that later transfers fail fast instead of queueing forever.
      for (auto& x : xfers_)
        if (!x.done) {
          auto& serving = x.item.is_send ? ci_->send_serving : ci_->recv_serving;
          if (serving[(size_t)x.item.peer].load() == x.ticket) serving[(size_t)x.item.peer].store(x.ticket + 1);
        }
    }
    publish_outcome();
    return PEAction::complete;
  }

  const NetMesh& mesh_;
  const char* name_;
  std::vector<Xfer> xfers_;
  std::string self_error_;
};

}  // namespace

HostState* make_net_collective(HostCommunicator::Impl* ci, CollArgs&& args, Request req, uint64_t seq) {
  return new NetCollState(ci, std::move(args), std::move(req), seq);
}

HostState* make_net_p2p(HostCommunicator::Impl* ci, std::vector<P2PItem>&& items, Request req, const char* name) {
  return new NetP2PState(ci, std::move(items), std::move(req), name);
}

}  // namespace host
}  // namespace internal
}  // namespace Al
