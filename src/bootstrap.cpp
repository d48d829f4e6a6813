// Unix-socket control plane (see al/bootstrap.hpp).
#include "al/bootstrap.hpp"

#include <errno.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <thread>

#include "al/util/utils.hpp"

namespace Al {
namespace internal {

namespace {

struct EnvRank { int rank = 0, size = 1, local = -1; std::string key; };

bool first_env(std::initializer_list<const char*> names, long& out) {
  for (const char* n : names) {
    const char* v = getenv(n);
    if (v && *v) { out = strtol(v, nullptr, 10); return true; }
  }
  return false;
}

EnvRank discover() {
  EnvRank e;
  long v;
  if (first_env({"AL_RANK", "RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK", "SLURM_PROCID", "FLUX_TASK_RANK",
                 "MV2_COMM_WORLD_RANK"}, v)) e.rank = (int)v;
  if (first_env({"AL_WORLD_SIZE", "WORLD_SIZE", "OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "SLURM_NTASKS",
                 "FLUX_JOB_SIZE", "MV2_COMM_WORLD_SIZE"}, v)) e.size = (int)v;
  if (first_env({"AL_LOCAL_RANK", "LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID",
                 "FLUX_TASK_LOCAL_ID", "MV2_COMM_WORLD_LOCAL_RANK"}, v)) e.local = (int)v;
  if (e.local < 0) e.local = e.rank;
  std::string key = env_str("AL_JOB_KEY");
  if (key.empty() && getenv("MASTER_PORT"))
    key = env_str("MASTER_ADDR", "127.0.0.1") + ":" + env_str("MASTER_PORT");
  if (key.empty()) key = env_str("TORCHELASTIC_RUN_ID");
  if (key.empty()) key = env_str("SLURM_JOB_ID");
  if (key.empty()) key = env_str("FLUX_JOB_ID");
  if (key.empty()) key = "solo-" + std::to_string(getpid());
  e.key = key;
  return e;
}

// Abstract-namespace address: no file is left behind when a rank dies.
socklen_t make_addr(sockaddr_un& a, const std::string& key, int rank) {
  memset(&a, 0, sizeof(a));
  a.sun_family = AF_UNIX;
  std::string name = "al_b200/" + key + "/" + std::to_string(rank);
  if (name.size() + 2 > sizeof(a.sun_path)) {
    // Keep the tail (it holds the port and the rank, which make the name unique).
    name = name.substr(name.size() - (sizeof(a.sun_path) - 2));
  }
  a.sun_path[0] = '\0';
  memcpy(a.sun_path + 1, name.data(), name.size());
  return (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
}

double timeout_s(const BootstrapFaults& f) {
  if (f.recv_timeout_s >= 0) return f.recv_timeout_s;
  return (double)env_long("AL_BOOTSTRAP_TIMEOUT_S", 120);
}

void write_all(int fd, const void* buf, size_t n) {
  const char* p = (const char*)buf;
  while (n) {
    ssize_t w = ::send(fd, p, n, MSG_NOSIGNAL);
    if (w < 0) {
      if (errno == EINTR) continue;
      throw_al_exception("bootstrap send failed: ", strerror(errno));
    }
    p += w;
    n -= (size_t)w;
  }
}

void read_all(int fd, void* buf, size_t n, double tmo_s, int peer) {
  char* p = (char*)buf;
  const double deadline = get_time() + tmo_s;
  while (n) {
    pollfd pf{fd, POLLIN, 0};
    double left = deadline - get_time();
    if (left <= 0) throw_al_exception("bootstrap: timed out waiting for rank ", peer);
    int pr = ::poll(&pf, 1, (int)std::min(left * 1000.0 + 1, 1000.0));
    if (pr < 0) {
      if (errno == EINTR) continue;
      throw_al_exception("bootstrap poll failed: ", strerror(errno));
    }
    if (pr == 0) continue;
    ssize_t r = ::recv(fd, p, n, 0);
    if (r == 0) throw_al_exception("bootstrap: rank ", peer, " closed the connection");
    if (r < 0) {
      if (errno == EINTR || errno == EAGAIN) continue;
      throw_al_exception("bootstrap recv failed: ", strerror(errno));
    }
    p += r;
    n -= (size_t)r;
  }
}

}  // namespace

std::unique_ptr<World> World::from_env() {
  EnvRank e = discover();
  return connect(e.rank, e.size, e.local, e.key);
}

std::unique_ptr<World> World::connect(int rank, int size, int local_rank, const std::string& key) {
  if (size < 1 || rank < 0 || rank >= size) throw_al_exception("invalid rank ", rank, " of ", size);
  std::unique_ptr<World> w(new World());
  w->rank_ = rank;
  w->size_ = size;
  w->local_rank_ = local_rank;
  w->local_size_ = size;  // single-host control plane: every rank is node-local
  w->key_ = key;
  w->socks_.assign((size_t)size, -1);
  if (size == 1) return w;

  const double tmo = timeout_s(w->faults);
  // Listen for the higher ranks.
  w->listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (w->listen_fd_ < 0) throw_al_exception("socket(): ", strerror(errno));
  sockaddr_un addr;
  socklen_t len = make_addr(addr, key, rank);
  if (::bind(w->listen_fd_, (sockaddr*)&addr, len) != 0)
    throw_al_exception("bootstrap bind failed for rank ", rank, " (job key '", key,
                       "' already in use?): ", strerror(errno));
  if (::listen(w->listen_fd_, size) != 0) throw_al_exception("listen(): ", strerror(errno));

  // Connect to the lower ranks (retry until they are listening).
  for (int peer = 0; peer < rank; ++peer) {
    const double deadline = get_time() + tmo;
    int fd = -1;
    for (;;) {
      fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
      if (fd < 0) throw_al_exception("socket(): ", strerror(errno));
      sockaddr_un pa;
      socklen_t pl = make_addr(pa, key, peer);
      if (::connect(fd, (sockaddr*)&pa, pl) == 0) break;
      ::close(fd);
      fd = -1;
      if (get_time() > deadline)
        throw_al_exception("bootstrap: rank ", rank, " could not reach rank ", peer, " within ", tmo, " s");
      std::this_thread::sleep_for(std::chrono::milliseconds(2));
    }
    int32_t me = rank;
    write_all(fd, &me, sizeof(me));
    w->socks_[(size_t)peer] = fd;
  }
  // Accept the higher ranks.
  for (int k = rank + 1; k < size; ++k) {
    const double deadline = get_time() + tmo;
    int fd = -1;
    for (;;) {
      pollfd pf{w->listen_fd_, POLLIN, 0};
      int pr = ::poll(&pf, 1, 200);
      if (pr > 0) {
        fd = ::accept4(w->listen_fd_, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd >= 0) break;
        if (errno != EINTR && errno != EAGAIN) throw_al_exception("accept(): ", strerror(errno));
      }
      if (get_time() > deadline)
        throw_al_exception("bootstrap: rank ", rank, " timed out waiting for ", size - k,
                           " higher rank(s) to connect");
    }
    int32_t who = -1;
    read_all(fd, &who, sizeof(who), tmo, -1);
    if (who <= rank || who >= size || w->socks_[(size_t)who] != -1)
      throw_al_exception("bootstrap: unexpected connection from rank ", who);
    w->socks_[(size_t)who] = fd;
  }
  return w;
}

World::~World() {
  for (int fd : socks_)
    if (fd >= 0) ::close(fd);
  if (listen_fd_ >= 0) ::close(listen_fd_);
}

void World::send(int peer, const void* buf, size_t bytes) {
  if (peer == rank_) throw_al_exception("bootstrap send to self");
  if (faults.drops_left > 0 && faults.drop_send_to == peer) {
    --faults.drops_left;
    return;  // injected fault: the message vanishes
  }
  write_all(socks_.at((size_t)peer), buf, bytes);
}

void World::recv(int peer, void* buf, size_t bytes) {
  if (peer == rank_) throw_al_exception("bootstrap recv from self");
  read_all(socks_.at((size_t)peer), buf, bytes, timeout_s(faults), peer);
}

void World::send_fd(int peer, int fd) {
  char byte = 'F';
  iovec iov{&byte, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  memset(ctrl, 0, sizeof(ctrl));
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  c->cmsg_level = SOL_SOCKET;
  c->cmsg_type = SCM_RIGHTS;
  c->cmsg_len = CMSG_LEN(sizeof(int));
  memcpy(CMSG_DATA(c), &fd, sizeof(int));
  for (;;) {
    ssize_t r = ::sendmsg(socks_.at((size_t)peer), &msg, MSG_NOSIGNAL);
    if (r == 1) return;
    if (r < 0 && errno == EINTR) continue;
    throw_al_exception("bootstrap send_fd failed: ", strerror(errno));
  }
}

int World::recv_fd(int peer) {
  const double deadline = get_time() + timeout_s(faults);
  const int sock = socks_.at((size_t)peer);
  for (;;) {
    pollfd pf{sock, POLLIN, 0};
    int pr = ::poll(&pf, 1, 200);
    if (pr > 0) break;
    if (get_time() > deadline) throw_al_exception("bootstrap: timed out waiting for a descriptor from rank ", peer);
  }
  char byte = 0;
  iovec iov{&byte, 1};
  alignas(cmsghdr) char ctrl[CMSG_SPACE(sizeof(int))];
  msghdr msg{};
  msg.msg_iov = &iov;
  msg.msg_iovlen = 1;
  msg.msg_control = ctrl;
  msg.msg_controllen = sizeof(ctrl);
  for (;;) {
    ssize_t r = ::recvmsg(sock, &msg, MSG_CMSG_CLOEXEC);
    if (r == 1) break;
    if (r < 0 && errno == EINTR) continue;
    throw_al_exception("bootstrap recv_fd failed: ", r == 0 ? "peer closed" : strerror(errno));
  }
  cmsghdr* c = CMSG_FIRSTHDR(&msg);
  if (!c || c->cmsg_level != SOL_SOCKET || c->cmsg_type != SCM_RIGHTS)
    throw_al_exception("bootstrap recv_fd: no descriptor attached");
  int fd;
  memcpy(&fd, CMSG_DATA(c), sizeof(int));
  return fd;
}

// ---------------------------------------------------------------------------

Group::Group(World* w, std::vector<int> members) : world_(w), members_(std::move(members)) {
  auto it = std::find(members_.begin(), members_.end(), w->rank());
  if (it == members_.end()) throw_al_exception("this rank is not a member of the group");
  me_ = (int)(it - members_.begin());
}

Group Group::world_group(World* w) {
  std::vector<int> m((size_t)w->size());
  for (int i = 0; i < w->size(); ++i) m[(size_t)i] = i;
  return Group(w, std::move(m));
}

void Group::allgather(const void* in, void* out, size_t bytes) const {
  std::lock_guard<std::mutex> g(world_->collective_mutex());
  char* o = (char*)out;
  if (in != o + (size_t)me_ * bytes) memcpy(o + (size_t)me_ * bytes, in, bytes);
  if (bytes == 0) return;
  // Pairwise exchange in increasing peer order; in each pair the lower rank
  // sends first, so no cycle of blocked senders can form.
  for (int r = 0; r < size(); ++r) {
    if (r == me_) continue;
    const int peer = members_[(size_t)r];
    if (me_ < r) {
      world_->send(peer, o + (size_t)me_ * bytes, bytes);
      world_->recv(peer, o + (size_t)r * bytes, bytes);
    } else {
      world_->recv(peer, o + (size_t)r * bytes, bytes);
      world_->send(peer, o + (size_t)me_ * bytes, bytes);
    }
  }
}

void Group::bcast(void* buf, size_t bytes, int root) const {
  std::lock_guard<std::mutex> g(world_->collective_mutex());
  if (bytes == 0) return;
  if (me_ == root) {
    for (int r = 0; r < size(); ++r)
      if (r != me_) world_->send(members_[(size_t)r], buf, bytes);
  } else {
    world_->recv(members_[(size_t)root], buf, bytes);
  }
}

void Group::barrier() const {
  std::vector<char> tmp((size_t)size());
  char one = 1;
  allgather(&one, tmp.data(), 1);
}

std::vector<int> Group::allgather_fd(int fd) const {
  std::lock_guard<std::mutex> g(world_->collective_mutex());
  std::vector<int> fds((size_t)size(), -1);
  fds[(size_t)me_] = ::dup(fd);
  for (int r = 0; r < size(); ++r) {
    if (r == me_) continue;
    const int peer = members_[(size_t)r];
    if (me_ < r) {
      world_->send_fd(peer, fd);
      fds[(size_t)r] = world_->recv_fd(peer);
    } else {
      fds[(size_t)r] = world_->recv_fd(peer);
      world_->send_fd(peer, fd);
    }
  }
  return fds;
}

Group Group::split(int color, int key) const {
  struct Entry { int color, key, old_rank, world_rank; };
  Entry mine{color, key, me_, world_->rank()};
  std::vector<Entry> all((size_t)size());
  allgather(&mine, all.data(), sizeof(Entry));
  std::vector<Entry> same;
  for (auto& e : all)
    if (e.color == color) same.push_back(e);
  std::stable_sort(same.begin(), same.end(), [](const Entry& a, const Entry& b) {
    return a.key != b.key ? a.key < b.key : a.old_rank < b.old_rank;
  });
  std::vector<int> members;
  for (auto& e : same) members.push_back(e.world_rank);
  return Group(world_, std::move(members));
}

uint64_t Group::agree_on_id() const {
  // The group's first member proposes; ids embed its world rank so that
  // disjoint groups created concurrently never collide.
  static std::atomic<uint64_t> counter{1};
  uint64_t id = 0;
  if (me_ == 0) id = ((uint64_t)world_->rank() << 40) | counter.fetch_add(1);
  bcast(&id, sizeof(id), 0);
  return id;
}

}  // namespace internal
}  // namespace Al
