// Socket control plane: Unix-domain sockets within a node, TCP between nodes (see al/bootstrap.hpp).
#include "al/bootstrap.hpp"

#include <arpa/inet.h>
#include <errno.h>
#include <netdb.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <set>
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
  return env_double("AL_BOOTSTRAP_TIMEOUT_S", 120.0);
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

// ---- TCP helpers -------------------------------------------------------------

int tcp_listen(int port, int backlog, int* bound_port) {
  int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) throw_al_exception("socket(): ", strerror(errno));
  int one = 1;
  ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_addr.s_addr = htonl(INADDR_ANY);
  a.sin_port = htons((uint16_t)port);
  if (::bind(fd, (sockaddr*)&a, sizeof(a)) != 0) {
    const int e = errno;
    ::close(fd);
    throw_al_exception("bootstrap: cannot bind TCP port ", port, ": ", strerror(e));
  }
  if (::listen(fd, backlog) != 0) {
    const int e = errno;
    ::close(fd);
    throw_al_exception("listen(): ", strerror(e));
  }
  socklen_t len = sizeof(a);
  if (bound_port && ::getsockname(fd, (sockaddr*)&a, &len) == 0) *bound_port = ntohs(a.sin_port);
  return fd;
}

/** Numeric IPv4 address of `host` (a name or an address). */
std::string resolve_ipv4(const std::string& host) {
  addrinfo hints{};
  hints.ai_family = AF_INET;
  hints.ai_socktype = SOCK_STREAM;
  addrinfo* res = nullptr;
  if (::getaddrinfo(host.c_str(), nullptr, &hints, &res) != 0 || !res)
    throw_al_exception("bootstrap: cannot resolve '", host, "'");
  char buf[INET_ADDRSTRLEN] = {0};
  ::inet_ntop(AF_INET, &((sockaddr_in*)res->ai_addr)->sin_addr, buf, sizeof(buf));
  ::freeaddrinfo(res);
  return buf;
}

/** Connects to ip:port, retrying until the deadline; returns -1 when it passed. */
int tcp_connect_retry(const std::string& ip, int port, double deadline) {
  sockaddr_in a{};
  a.sin_family = AF_INET;
  a.sin_port = htons((uint16_t)port);
  if (::inet_pton(AF_INET, ip.c_str(), &a.sin_addr) != 1) throw_al_exception("bootstrap: bad address '", ip, "'");
  for (;;) {
    int fd = ::socket(AF_INET, SOCK_STREAM | SOCK_CLOEXEC, 0);
    if (fd < 0) throw_al_exception("socket(): ", strerror(errno));
    if (::connect(fd, (sockaddr*)&a, sizeof(a)) == 0) {
      int one = 1;
      ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
      return fd;
    }
    ::close(fd);
    if (get_time() > deadline) return -1;
    std::this_thread::sleep_for(std::chrono::milliseconds(5));
  }
}

struct Hello { int32_t rank; int32_t port; char node[64]; };
struct TableEntry { char node[64]; char ip[48]; int32_t port; };

bool launcher_reports_several_nodes(const EnvRank& e) {
  long v;
  if (first_env({"AL_NNODES", "SLURM_NNODES", "SLURM_JOB_NUM_NODES", "OMPI_MCA_orte_num_nodes"}, v) && v > 1) return true;
  if (first_env({"LOCAL_WORLD_SIZE", "OMPI_COMM_WORLD_LOCAL_SIZE", "SLURM_NTASKS_PER_NODE"}, v) && v > 0 && v < e.size)
    return true;
  return false;
}

}  // namespace

int bootstrap_tcp_listen(int* port) { return tcp_listen(0, 128, port); }
int bootstrap_tcp_connect(const std::string& ip, int port, double timeout_s) {
  return tcp_connect_retry(ip, port, get_time() + timeout_s);
}

std::unique_ptr<World> World::from_env() {
  EnvRank e = discover();
  const std::string mode = env_str("AL_TRANSPORT", "auto");
  if (mode != "auto" && mode != "unix" && mode != "tcp")
    throw_al_exception("AL_TRANSPORT must be auto, unix or tcp (got '", mode, "')");
  bool tcp = mode == "tcp";
  if (mode == "auto") tcp = getenv("MASTER_ADDR") != nullptr && launcher_reports_several_nodes(e);
  if (!tcp || e.size == 1) return connect(e.rank, e.size, e.local, e.key);
  const std::string master = env_str("MASTER_ADDR", "127.0.0.1");
  const long port = env_long("AL_MASTER_PORT", env_long("MASTER_PORT", 29400) + 1);
  std::string node = env_str("AL_NODE_ID");
  if (node.empty()) {
    char host[64] = {0};
    ::gethostname(host, sizeof(host) - 1);
    node = host;
  }
  long hint;
  const bool has_local = first_env({"AL_LOCAL_RANK", "LOCAL_RANK", "OMPI_COMM_WORLD_LOCAL_RANK", "SLURM_LOCALID",
                                    "FLUX_TASK_LOCAL_ID", "MV2_COMM_WORLD_LOCAL_RANK"}, hint);
  return connect_tcp(e.rank, e.size, has_local ? (int)hint : -1, e.key, master, (int)port, node);
}

namespace {
int unix_listen(const std::string& key, int rank, int size) {
  int fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
  if (fd < 0) throw_al_exception("socket(): ", strerror(errno));
  sockaddr_un addr;
  socklen_t len = make_addr(addr, key, rank);
  if (::bind(fd, (sockaddr*)&addr, len) != 0) {
    const int e = errno;
    ::close(fd);
    throw_al_exception("bootstrap bind failed for rank ", rank, " (job key '", key, "' already in use?): ", strerror(e));
  }
  if (::listen(fd, size) != 0) {
    const int e = errno;
    ::close(fd);
    throw_al_exception("listen(): ", strerror(e));
  }
  return fd;
}
}  // namespace

std::unique_ptr<World> World::connect(int rank, int size, int local_rank, const std::string& key) {
  if (size < 1 || rank < 0 || rank >= size) throw_al_exception("invalid rank ", rank, " of ", size);
  std::unique_ptr<World> w(new World());
  w->rank_ = rank;
  w->size_ = size;
  w->local_rank_ = local_rank;
  w->local_size_ = size;  // single-host control plane: every rank is node-local
  w->key_ = key;
  w->socks_.assign((size_t)size, -1);
  w->nodes_.assign((size_t)size, "localhost");
  w->addrs_.assign((size_t)size, "127.0.0.1");
  if (size == 1) return w;
  w->listen_fd_ = unix_listen(key, rank, size);
  w->mesh({}, timeout_s(w->faults));
  return w;
}

std::unique_ptr<World> World::connect_tcp(int rank, int size, int local_rank_hint, const std::string& key,
                                          const std::string& master_addr, int master_port,
                                          const std::string& node_id) {
  if (size < 1 || rank < 0 || rank >= size) throw_al_exception("invalid rank ", rank, " of ", size);
  std::unique_ptr<World> w(new World());
  w->rank_ = rank;
  w->size_ = size;
  w->key_ = key;
  w->socks_.assign((size_t)size, -1);
  const double tmo = timeout_s(w->faults);
  w->listen_fd_ = unix_listen(key, rank, size);
  int my_port = 0;
  w->tcp_listen_fd_ = tcp_listen(0, size, &my_port);

  // Rendezvous: rank 0 gathers (node, address, port) of every rank and returns the table.
  std::vector<TableEntry> table((size_t)size);
  memset(table.data(), 0, table.size() * sizeof(TableEntry));
  const std::string master_ip = resolve_ipv4(master_addr);
  if (rank == 0) {
    // A launcher may hand over the rendezvous socket already listening (no window in which
    // another process could take the port); otherwise listen on the agreed port.
    const long inherited = env_long("AL_MASTER_FD", -1);
    int mfd = inherited >= 0 ? (int)inherited : tcp_listen(master_port, size, nullptr);
    std::vector<int> fds;
    auto close_all = [&] { for (int f : fds) ::close(f); ::close(mfd); };
    snprintf(table[0].node, sizeof(table[0].node), "%s", node_id.c_str());
    snprintf(table[0].ip, sizeof(table[0].ip), "%s", master_ip.c_str());
    table[0].port = my_port;
    const double deadline = get_time() + tmo;
    try {
      for (int k = 1; k < size; ++k) {
        int fd = -1;
        sockaddr_in from{};
        socklen_t flen = sizeof(from);
        for (;;) {
          pollfd pf{mfd, POLLIN, 0};
          if (::poll(&pf, 1, 200) > 0) {
            fd = ::accept4(mfd, (sockaddr*)&from, &flen, SOCK_CLOEXEC);
            if (fd >= 0) break;
            if (errno != EINTR && errno != EAGAIN) throw_al_exception("accept(): ", strerror(errno));
          }
          if (get_time() > deadline)
            throw_al_exception("bootstrap: rank 0 timed out waiting for ", size - k, " rank(s) at the rendezvous port ",
                               master_port);
        }
        fds.push_back(fd);
        Hello h{};
        read_all(fd, &h, sizeof(h), tmo, -1);
        if (h.rank <= 0 || h.rank >= size || table[(size_t)h.rank].port != 0)
          throw_al_exception("bootstrap: unexpected rank ", h.rank, " at the rendezvous");
        TableEntry& t = table[(size_t)h.rank];
        h.node[sizeof(h.node) - 1] = 0;
        snprintf(t.node, sizeof(t.node), "%s", h.node);
        ::inet_ntop(AF_INET, &from.sin_addr, t.ip, sizeof(t.ip));
        t.port = h.port;
      }
      for (int fd : fds) write_all(fd, table.data(), table.size() * sizeof(TableEntry));
    } catch (...) {
      close_all();
      throw;
    }
    close_all();
  } else {
    int fd = tcp_connect_retry(master_ip, master_port, get_time() + tmo);
    if (fd < 0)
      throw_al_exception("bootstrap: rank ", rank, " could not reach the rendezvous at ", master_addr, ":", master_port,
                         " within ", tmo, " s");
    Hello h{};
    h.rank = rank;
    h.port = my_port;
    snprintf(h.node, sizeof(h.node), "%s", node_id.c_str());
    try {
      write_all(fd, &h, sizeof(h));
      read_all(fd, table.data(), table.size() * sizeof(TableEntry), tmo, 0);
    } catch (...) {
      ::close(fd);
      throw;
    }
    ::close(fd);
  }
  std::vector<int> ports((size_t)size);
  std::set<std::string> distinct;
  for (int r = 0; r < size; ++r) {
    w->nodes_.push_back(table[(size_t)r].node);
    w->addrs_.push_back(table[(size_t)r].ip);
    ports[(size_t)r] = table[(size_t)r].port;
    distinct.insert(table[(size_t)r].node);
  }
  w->num_nodes_ = (int)distinct.size();
  int local_size = 0, local_rank = 0;
  for (int r = 0; r < size; ++r)
    if (w->nodes_[(size_t)r] == w->nodes_[(size_t)rank]) {
      if (r < rank) ++local_rank;
      ++local_size;
    }
  w->local_size_ = local_size;
  w->local_rank_ = (local_rank_hint >= 0 && local_rank_hint < local_size) ? local_rank_hint : local_rank;
  w->mesh(ports, tmo);
  return w;
}

/** Full mesh: the higher rank of a pair connects, over a Unix socket within a node and TCP otherwise. */
void World::mesh(const std::vector<int>& tcp_ports, double tmo) {
  const int rank = rank_, size = size_;
  for (int peer = 0; peer < rank; ++peer) {
    const double deadline = get_time() + tmo;
    int fd = -1;
    if (same_node(peer)) {
      for (;;) {
        fd = ::socket(AF_UNIX, SOCK_STREAM | SOCK_CLOEXEC, 0);
        if (fd < 0) throw_al_exception("socket(): ", strerror(errno));
        sockaddr_un pa;
        socklen_t pl = make_addr(pa, key_, peer);
        if (::connect(fd, (sockaddr*)&pa, pl) == 0) break;
        ::close(fd);
        fd = -1;
        if (get_time() > deadline)
          throw_al_exception("bootstrap: rank ", rank, " could not reach rank ", peer, " within ", tmo, " s");
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
      }
    } else {
      fd = tcp_connect_retry(addrs_[(size_t)peer], tcp_ports.at((size_t)peer), deadline);
      if (fd < 0)
        throw_al_exception("bootstrap: rank ", rank, " could not reach rank ", peer, " at ", addrs_[(size_t)peer], ":",
                           tcp_ports[(size_t)peer], " within ", tmo, " s");
    }
    int32_t me = rank;
    write_all(fd, &me, sizeof(me));
    socks_[(size_t)peer] = fd;
  }
  // Accept the higher ranks on whichever listening socket they arrive.
  for (int k = rank + 1; k < size; ++k) {
    const double deadline = get_time() + tmo;
    int fd = -1;
    for (;;) {
      pollfd pf[2] = {{listen_fd_, POLLIN, 0}, {tcp_listen_fd_, POLLIN, 0}};
      const int n = tcp_listen_fd_ >= 0 ? 2 : 1;
      if (::poll(pf, (nfds_t)n, 200) > 0) {
        const int lfd = (pf[0].revents & POLLIN) ? listen_fd_ : tcp_listen_fd_;
        fd = ::accept4(lfd, nullptr, nullptr, SOCK_CLOEXEC);
        if (fd >= 0) {
          if (lfd == tcp_listen_fd_) {
            int one = 1;
            ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
          }
          break;
        }
        if (errno != EINTR && errno != EAGAIN) throw_al_exception("accept(): ", strerror(errno));
      }
      if (get_time() > deadline)
        throw_al_exception("bootstrap: rank ", rank, " timed out waiting for ", size - k,
                           " higher rank(s) to connect");
    }
    int32_t who = -1;
    read_all(fd, &who, sizeof(who), tmo, -1);
    if (who <= rank || who >= size || socks_[(size_t)who] != -1)
      throw_al_exception("bootstrap: unexpected connection from rank ", who);
    socks_[(size_t)who] = fd;
  }
}

int World::node_index(int rank) const {
  int idx = 0;
  for (int r = 0; r < size_; ++r) {
    if (nodes_[(size_t)r] == nodes_.at((size_t)rank)) return idx;
    bool first = true;  // r opens a new node unless an earlier rank shares its name
    for (int q = 0; q < r; ++q)
      if (nodes_[(size_t)q] == nodes_[(size_t)r]) { first = false; break; }
    if (first) ++idx;
  }
  return idx;
}

World::~World() {
  for (int fd : socks_)
    if (fd >= 0) ::close(fd);
  if (listen_fd_ >= 0) ::close(listen_fd_);
  if (tcp_listen_fd_ >= 0) ::close(tcp_listen_fd_);
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

bool World::peer_alive(int peer) const {
  if (peer == rank_) return true;
  const int fd = socks_.at((size_t)peer);
  if (fd < 0) return true;
  pollfd pf{fd, POLLIN | POLLRDHUP, 0};
  if (::poll(&pf, 1, 0) <= 0) return true;
  if (pf.revents & (POLLRDHUP | POLLHUP | POLLERR | POLLNVAL)) return false;
  // Readable: either a control message is waiting (alive) or the stream ended (a read of 0 bytes).
  char c;
  const ssize_t n = ::recv(fd, &c, 1, MSG_PEEK | MSG_DONTWAIT);
  return n != 0;
}

void World::send_fd(int peer, int fd) {
  if (!same_node(peer))
    throw_al_exception("rank ", peer, " is on another node (", node_of(peer), "): descriptors cannot be passed to it");
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
  if (!same_node(peer))
    throw_al_exception("rank ", peer, " is on another node (", node_of(peer), "): descriptors cannot be passed from it");
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

bool Group::single_node() const {
  for (int m : members_)
    if (!world_->same_node(m)) return false;
  return true;
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
