// Implementation of the single-node MPI stand-in declared in mpi.h.
//
// Transport: one non-blocking Unix-domain stream socket per pair of processes (abstract
// names, so nothing is left in the file system).  Every message is a 24-byte header
// {context, tag, byte count} followed by the payload.  A send completes when its bytes are in
// the socket; a receive matches on (source, context, tag) in posting order, arrivals without
// a posted receive are kept in an "unexpected" list.  Every call that waits drives the same
// progress() routine, which writes what can be written and reads what has arrived, so two
// ranks that send large messages to each other cannot block one another.
//
// Collectives are schedules of point-to-point transfers on a private context of the
// communicator plus a completion step (a reduction in rank order, or nothing).  The
// non-blocking forms return such a schedule as the request; the blocking forms wait for it.
// With at most a handful of ranks on one machine every collective is a direct exchange: there
// are no trees or rings.
//
// Thread safety: one mutex around every entry point, released between polls of a blocking
// wait (MPI_THREAD_MULTIPLE is what Aluminum asks for: its progress thread calls MPI while
// the main thread may too, src/mpi_impl.cpp:150-165 of the reference).
#include "mpi.h"

#include <errno.h>
#include <fcntl.h>
#include <poll.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/socket.h>
#include <sys/stat.h>
#include <sys/un.h>
#include <time.h>
#include <unistd.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <functional>
#include <list>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

namespace {

// ------------------------------------------------------------------------------------------
// state
// ------------------------------------------------------------------------------------------
std::recursive_mutex g_mu;
bool g_initialized = false, g_finalized = false;
int g_rank = 0, g_size = 1;
int g_tag_ub = (1 << 30) - 1;
int g_next_ctx = 16;
double g_timeout_s = 120.0;

[[noreturn]] void die(const char* what) {
  fprintf(stderr, "[mpi_shim rank %d] fatal: %s\n", g_rank, what);
  fflush(stderr);
  _exit(70);
}

double now_s() {
  timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

struct Header {
  int32_t ctx;
  int32_t tag;
  uint64_t nbytes;
  uint64_t pad;
};

struct Req {
  enum Kind { kFree, kSend, kRecv, kColl } kind = kFree;
  bool done = false;
  // send
  Header hdr{};
  const char* sdata = nullptr;
  size_t written = 0;  // header + payload bytes written
  std::vector<char> owned;
  // recv
  char* rdata = nullptr;
  size_t rcap = 0;
  int src_world = -1, ctx = 0, tag = 0;
  MPI_Status st{};
  int comm_src = 0;  // rank of the source in the communicator (for the status)
  // collective schedule
  std::vector<int> children;
  std::function<void()> finish;
  std::vector<std::shared_ptr<std::vector<char>>> temps;
};

std::vector<Req> g_reqs(1);  // index 0 = MPI_REQUEST_NULL
std::vector<int> g_free_reqs;

int new_req(Req::Kind k) {
  int id;
  if (!g_free_reqs.empty()) { id = g_free_reqs.back(); g_free_reqs.pop_back(); }
  else { id = (int)g_reqs.size(); g_reqs.emplace_back(); }
  g_reqs[(size_t)id] = Req();
  g_reqs[(size_t)id].kind = k;
  return id;
}
void free_req(int id) {
  g_reqs[(size_t)id] = Req();
  g_free_reqs.push_back(id);
}

struct Unexpected {
  Header hdr;
  std::vector<char> data;
  bool complete = false;
};

struct Peer {
  int fd = -1;
  std::deque<int> out;          // send requests, in order
  // incoming parser
  Header in_hdr{};
  size_t in_hdr_got = 0;
  bool in_body = false;
  size_t in_body_got = 0;
  int in_req = 0;               // receive request the body goes to (0: into `in_unexp`)
  Unexpected* in_unexp = nullptr;
  std::list<int> posted;        // posted receives from this peer, in order
  std::list<Unexpected> unexpected;
};
std::vector<Peer> g_peers;

struct Comm {
  bool used = false;
  int ctx = 0;
  std::vector<int> ranks;  // world ranks
  int me = -1;
  unsigned coll_seq = 0;
};
std::vector<Comm> g_comms(3);

struct Group {
  bool used = false;
  std::vector<int> ranks;
  int me = MPI_UNDEFINED;
};
std::vector<Group> g_groups(2);

struct UserOp { bool used = false; MPI_User_function* fn = nullptr; };
std::vector<UserOp> g_ops(16);

// ------------------------------------------------------------------------------------------
// datatypes and reductions
// ------------------------------------------------------------------------------------------
enum Kind { I8, U8, I16, U16, I32, U32, I64, U64, F32, F64, F80, BOOL, NONE };
struct TypeInfo { size_t size; Kind kind; };
TypeInfo type_info(MPI_Datatype dt) {
  switch (dt) {
    case MPI_CHAR: return {1, I8};
    case MPI_SIGNED_CHAR: return {1, I8};
    case MPI_UNSIGNED_CHAR: return {1, U8};
    case MPI_BYTE: return {1, U8};
    case MPI_SHORT: return {2, I16};
    case MPI_UNSIGNED_SHORT: return {2, U16};
    case MPI_INT: return {4, I32};
    case MPI_UNSIGNED: return {4, U32};
    case MPI_LONG: return {sizeof(long), I64};
    case MPI_UNSIGNED_LONG: return {sizeof(unsigned long), U64};
    case MPI_LONG_LONG_INT: return {8, I64};
    case MPI_UNSIGNED_LONG_LONG: return {8, U64};
    case MPI_FLOAT: return {4, F32};
    case MPI_DOUBLE: return {8, F64};
    case MPI_LONG_DOUBLE: return {sizeof(long double), F80};
    case MPI_INT8_T: return {1, I8};
    case MPI_UINT8_T: return {1, U8};
    case MPI_INT16_T: return {2, I16};
    case MPI_UINT16_T: return {2, U16};
    case MPI_INT32_T: return {4, I32};
    case MPI_UINT32_T: return {4, U32};
    case MPI_INT64_T: return {8, I64};
    case MPI_UINT64_T: return {8, U64};
    case MPI_C_BOOL: return {1, BOOL};
    case MPI_CXX_BOOL: return {sizeof(bool), BOOL};
    case MPI_WCHAR: return {sizeof(wchar_t), I32};
    case MPI_AINT: return {sizeof(MPI_Aint), I64};
    case MPI_COUNT: return {8, I64};
    case MPI_OFFSET: return {8, I64};
    default: die("unknown datatype");
  }
}

template <typename T, bool Int>
struct Apply {
  static void run(MPI_Op op, const T* in, T* io, size_t n) {
    for (size_t i = 0; i < n; ++i) {
      const T a = in[i], b = io[i];
      switch (op) {
        case MPI_SUM: io[i] = (T)(a + b); break;
        case MPI_PROD: io[i] = (T)(a * b); break;
        case MPI_MIN: io[i] = b < a ? b : a; break;
        case MPI_MAX: io[i] = a < b ? b : a; break;
        case MPI_LAND: io[i] = (T)((a != T(0)) && (b != T(0))); break;
        case MPI_LOR: io[i] = (T)((a != T(0)) || (b != T(0))); break;
        case MPI_LXOR: io[i] = (T)((a != T(0)) != (b != T(0))); break;
        default:
          if constexpr (Int) {
            if (op == MPI_BAND) io[i] = (T)(a & b);
            else if (op == MPI_BOR) io[i] = (T)(a | b);
            else if (op == MPI_BXOR) io[i] = (T)(a ^ b);
            else die("unknown reduction operator");
          } else {
            die("bitwise reduction on a floating-point type");
          }
      }
    }
  }
};

/** inout = in (op) inout, element-wise. */
void reduce_into(MPI_Op op, MPI_Datatype dt, const void* in, void* inout, size_t n) {
  if (op > MPI_BXOR) {
    const size_t idx = (size_t)op - 16;
    if (idx >= g_ops.size() || !g_ops[idx].used) die("invalid user-defined operator");
    // user functions take an int length: feed them in pieces
    const size_t esz = type_info(dt).size;
    size_t done = 0;
    while (done < n) {
      int len = (int)std::min<size_t>(n - done, 1u << 30);
      MPI_Datatype d = dt;
      g_ops[idx].fn((char*)in + done * esz, (char*)inout + done * esz, &len, &d);
      done += (size_t)len;
    }
    return;
  }
  switch (type_info(dt).kind) {
    case I8: Apply<int8_t, true>::run(op, (const int8_t*)in, (int8_t*)inout, n); break;
    case U8: Apply<uint8_t, true>::run(op, (const uint8_t*)in, (uint8_t*)inout, n); break;
    case I16: Apply<int16_t, true>::run(op, (const int16_t*)in, (int16_t*)inout, n); break;
    case U16: Apply<uint16_t, true>::run(op, (const uint16_t*)in, (uint16_t*)inout, n); break;
    case I32: Apply<int32_t, true>::run(op, (const int32_t*)in, (int32_t*)inout, n); break;
    case U32: Apply<uint32_t, true>::run(op, (const uint32_t*)in, (uint32_t*)inout, n); break;
    case I64: Apply<int64_t, true>::run(op, (const int64_t*)in, (int64_t*)inout, n); break;
    case U64: Apply<uint64_t, true>::run(op, (const uint64_t*)in, (uint64_t*)inout, n); break;
    case F32: Apply<float, false>::run(op, (const float*)in, (float*)inout, n); break;
    case F64: Apply<double, false>::run(op, (const double*)in, (double*)inout, n); break;
    case F80: Apply<long double, false>::run(op, (const long double*)in, (long double*)inout, n); break;
    case BOOL: Apply<uint8_t, true>::run(op, (const uint8_t*)in, (uint8_t*)inout, n); break;
    default: die("reduction on an unsupported datatype");
  }
}

// ------------------------------------------------------------------------------------------
// progress
// ------------------------------------------------------------------------------------------
void complete_recv(Req& r, const Header& h, int src_world) {
  r.done = true;
  r.st.MPI_SOURCE = r.comm_src;
  r.st.MPI_TAG = h.tag;
  r.st.MPI_ERROR = MPI_SUCCESS;
  r.st.shim_bytes = (long long)h.nbytes;
  (void)src_world;
}

/** Write as much as the socket takes.  Returns true if something moved. */
bool pump_out(Peer& P) {
  bool moved = false;
  while (!P.out.empty()) {
    Req& r = g_reqs[(size_t)P.out.front()];
    const size_t total = sizeof(Header) + (size_t)r.hdr.nbytes;
    while (r.written < total) {
      const char* src;
      size_t len;
      if (r.written < sizeof(Header)) {
        src = (const char*)&r.hdr + r.written;
        len = sizeof(Header) - r.written;
      } else {
        src = r.sdata + (r.written - sizeof(Header));
        len = total - r.written;
      }
      const ssize_t n = ::send(P.fd, src, len, MSG_NOSIGNAL);
      if (n < 0) {
        if (errno == EAGAIN || errno == EWOULDBLOCK) return moved;
        if (errno == EINTR) continue;
        die("send to a peer failed (peer gone?)");
      }
      r.written += (size_t)n;
      moved = true;
    }
    r.done = true;
    P.out.pop_front();
  }
  return moved;
}

bool pump_in(Peer& P, int src_world) {
  bool moved = false;
  for (;;) {
    if (!P.in_body) {
      const ssize_t n = ::recv(P.fd, (char*)&P.in_hdr + P.in_hdr_got, sizeof(Header) - P.in_hdr_got, 0);
      if (n < 0) {
        if (errno == EAGAIN || errno == EWOULDBLOCK) return moved;
        if (errno == EINTR) continue;
        die("recv from a peer failed");
      }
      if (n == 0) return moved;  // peer closed; only fatal if somebody still waits (time-out reports it)
      moved = true;
      P.in_hdr_got += (size_t)n;
      if (P.in_hdr_got < sizeof(Header)) continue;
      // header complete: match
      P.in_hdr_got = 0;
      P.in_body = true;
      P.in_body_got = 0;
      P.in_req = 0;
      P.in_unexp = nullptr;
      for (auto it = P.posted.begin(); it != P.posted.end(); ++it) {
        Req& r = g_reqs[(size_t)*it];
        if (r.ctx == P.in_hdr.ctx && r.tag == P.in_hdr.tag) {
          if (P.in_hdr.nbytes > r.rcap) die("message longer than the posted receive buffer");
          P.in_req = *it;
          P.posted.erase(it);
          break;
        }
      }
      if (!P.in_req) {
        P.unexpected.emplace_back();
        P.in_unexp = &P.unexpected.back();
        P.in_unexp->hdr = P.in_hdr;
        P.in_unexp->data.resize((size_t)P.in_hdr.nbytes);
      }
    }
    // body
    const size_t total = (size_t)P.in_hdr.nbytes;
    while (P.in_body_got < total) {
      char* dst = P.in_req ? g_reqs[(size_t)P.in_req].rdata : P.in_unexp->data.data();
      const ssize_t n = ::recv(P.fd, dst + P.in_body_got, total - P.in_body_got, 0);
      if (n < 0) {
        if (errno == EAGAIN || errno == EWOULDBLOCK) return moved;
        if (errno == EINTR) continue;
        die("recv from a peer failed");
      }
      if (n == 0) return moved;
      moved = true;
      P.in_body_got += (size_t)n;
    }
    if (P.in_req) complete_recv(g_reqs[(size_t)P.in_req], P.in_hdr, src_world);
    else P.in_unexp->complete = true;
    P.in_body = false;
  }
}

bool progress() {
  bool moved = false;
  for (int r = 0; r < g_size; ++r) {
    if (r == g_rank) continue;
    Peer& P = g_peers[(size_t)r];
    if (P.fd < 0) continue;
    moved |= pump_out(P);
    moved |= pump_in(P, r);
  }
  return moved;
}

bool req_done(int id) {
  Req& r = g_reqs[(size_t)id];
  if (r.done) return true;
  if (r.kind == Req::kColl) {
    for (int c : r.children)
      if (!req_done(c)) return false;
    for (int c : r.children) free_req(c);
    r.children.clear();
    if (r.finish) { r.finish(); r.finish = nullptr; }
    r.temps.clear();
    r.done = true;
    return true;
  }
  return false;
}

/** Block (dropping the lock between polls) until `pred` holds. */
template <typename Pred>
void wait_until(std::unique_lock<std::recursive_mutex>& lk, Pred pred, const char* what) {
  const double t0 = now_s();
  unsigned idle = 0;
  for (;;) {
    const bool moved = progress();
    if (pred()) return;
    if (moved) { idle = 0; continue; }
    lk.unlock();
    if (++idle < 200) sched_yield();
    else {
      pollfd fds[64];
      int n = 0;
      for (int r = 0; r < g_size && n < 64; ++r)
        if (r != g_rank && g_peers[(size_t)r].fd >= 0) { fds[n].fd = g_peers[(size_t)r].fd; fds[n].events = POLLIN; fds[n].revents = 0; ++n; }
      if (n) ::poll(fds, (nfds_t)n, 1);
      else usleep(100);
    }
    lk.lock();
    if ((idle & 1023) == 0 && now_s() - t0 > g_timeout_s) {
      fprintf(stderr, "[mpi_shim rank %d] no progress for %.0f s in %s\n", g_rank, g_timeout_s, what);
      die("time-out");
    }
  }
}

// ------------------------------------------------------------------------------------------
// point-to-point primitives on (world rank, context, tag)
// ------------------------------------------------------------------------------------------
int post_send(const void* buf, size_t nbytes, int dst_world, int ctx, int tag) {
  const int id = new_req(Req::kSend);
  Req& r = g_reqs[(size_t)id];
  r.hdr.ctx = ctx;
  r.hdr.tag = tag;
  r.hdr.nbytes = nbytes;
  r.sdata = (const char*)buf;
  if (dst_world == g_rank) {
    // self: hand over to a posted receive or park a copy
    Peer& P = g_peers[(size_t)g_rank];
    for (auto it = P.posted.begin(); it != P.posted.end(); ++it) {
      Req& q = g_reqs[(size_t)*it];
      if (q.ctx == ctx && q.tag == tag) {
        if (nbytes > q.rcap) die("self message longer than the posted receive buffer");
        if (nbytes) memcpy(q.rdata, buf, nbytes);
        complete_recv(q, r.hdr, g_rank);
        P.posted.erase(it);
        g_reqs[(size_t)id].done = true;
        return id;
      }
    }
    P.unexpected.emplace_back();
    Unexpected& u = P.unexpected.back();
    u.hdr = r.hdr;
    u.data.assign((const char*)buf, (const char*)buf + nbytes);
    u.complete = true;
    r.done = true;
    return id;
  }
  Peer& P = g_peers[(size_t)dst_world];
  if (P.fd < 0) die("send to an unconnected rank");
  P.out.push_back(id);
  pump_out(P);
  return id;
}

int post_recv(void* buf, size_t cap, int src_world, int ctx, int tag, int comm_src) {
  const int id = new_req(Req::kRecv);
  Req& r = g_reqs[(size_t)id];
  r.rdata = (char*)buf;
  r.rcap = cap;
  r.src_world = src_world;
  r.ctx = ctx;
  r.tag = tag;
  r.comm_src = comm_src;
  Peer& P = g_peers[(size_t)src_world];
  for (auto it = P.unexpected.begin(); it != P.unexpected.end(); ++it) {
    if (it->hdr.ctx != ctx || it->hdr.tag != tag) continue;
    if (!it->complete) {
      // the body of this message is still arriving into the unexpected buffer; wait for it
      // by leaving the request posted behind it: simplest is to finish the arrival first
      while (!it->complete) {
        if (!pump_in(P, src_world)) { sched_yield(); }
      }
    }
    if (it->hdr.nbytes > cap) die("message longer than the receive buffer");
    if (it->hdr.nbytes) memcpy(buf, it->data.data(), (size_t)it->hdr.nbytes);
    complete_recv(r, it->hdr, src_world);
    P.unexpected.erase(it);
    return id;
  }
  P.posted.push_back(id);
  return id;
}

Comm& comm_of(MPI_Comm c) {
  if (c <= 0 || (size_t)c >= g_comms.size() || !g_comms[(size_t)c].used) die("invalid communicator");
  return g_comms[(size_t)c];
}

MPI_Comm new_comm(int ctx, std::vector<int> ranks) {
  size_t id = 3;
  while (id < g_comms.size() && g_comms[id].used) ++id;
  if (id == g_comms.size()) g_comms.emplace_back();
  Comm& c = g_comms[id];
  c.used = true;
  c.ctx = ctx;
  c.ranks = std::move(ranks);
  c.me = -1;
  c.coll_seq = 0;
  for (size_t i = 0; i < c.ranks.size(); ++i)
    if (c.ranks[i] == g_rank) c.me = (int)i;
  return (MPI_Comm)id;
}

// ------------------------------------------------------------------------------------------
// collective schedules
// ------------------------------------------------------------------------------------------
struct Sched {
  Comm& c;
  int id;
  int tag;
  explicit Sched(Comm& comm) : c(comm), id(new_req(Req::kColl)), tag((int)(comm.coll_seq++ & 0x3fffffff)) {}
  Req& req() { return g_reqs[(size_t)id]; }
  void send(const void* buf, size_t nbytes, int dst) {
    const int child = post_send(buf, nbytes, c.ranks[(size_t)dst], c.ctx + 1, tag);
    g_reqs[(size_t)id].children.push_back(child);
  }
  void recv(void* buf, size_t nbytes, int src) {
    const int child = post_recv(buf, nbytes, c.ranks[(size_t)src], c.ctx + 1, tag, src);
    g_reqs[(size_t)id].children.push_back(child);
  }
  char* temp(size_t nbytes) {
    auto t = std::make_shared<std::vector<char>>(nbytes ? nbytes : 1);
    g_reqs[(size_t)id].temps.push_back(t);
    return t->data();
  }
  void on_finish(std::function<void()> f) { g_reqs[(size_t)id].finish = std::move(f); }
};

int wait_one(std::unique_lock<std::recursive_mutex>& lk, int id, MPI_Status* st, const char* what) {
  wait_until(lk, [&] { return req_done(id); }, what);
  if (st) *st = g_reqs[(size_t)id].st;
  free_req(id);
  return MPI_SUCCESS;
}

int sched_allreduce(Comm& c, const void* sendbuf, void* recvbuf, size_t count, MPI_Datatype dt, MPI_Op op) {
  const int p = (int)c.ranks.size();
  const size_t nb = count * type_info(dt).size;
  Sched s(c);
  // every rank receives every contribution and folds them in rank order: identical results everywhere
  char* all = s.temp(nb * (size_t)p);
  const void* mine = sendbuf == MPI_IN_PLACE ? recvbuf : sendbuf;
  if (nb) memcpy(all + (size_t)c.me * nb, mine, nb);
  for (int r = 0; r < p; ++r) {
    if (r == c.me) continue;
    s.recv(all + (size_t)r * nb, nb, r);
  }
  for (int r = 0; r < p; ++r) {
    if (r == c.me) continue;
    s.send(all + (size_t)c.me * nb, nb, r);
  }
  s.on_finish([=] {
    char* acc = all + (size_t)(p - 1) * nb;
    for (int r = p - 2; r >= 0; --r) reduce_into(op, dt, all + (size_t)r * nb, acc, count);
    if (nb) memcpy(recvbuf, acc, nb);
  });
  return s.id;
}

int sched_reduce(Comm& c, const void* sendbuf, void* recvbuf, size_t count, MPI_Datatype dt, MPI_Op op, int root) {
  const int p = (int)c.ranks.size();
  const size_t nb = count * type_info(dt).size;
  Sched s(c);
  if (c.me != root) {
    s.send(sendbuf, nb, root);
    return s.id;
  }
  char* all = s.temp(nb * (size_t)p);
  const void* mine = sendbuf == MPI_IN_PLACE ? recvbuf : sendbuf;
  if (nb) memcpy(all + (size_t)c.me * nb, mine, nb);
  for (int r = 0; r < p; ++r)
    if (r != c.me) s.recv(all + (size_t)r * nb, nb, r);
  s.on_finish([=] {
    char* acc = all + (size_t)(p - 1) * nb;
    for (int r = p - 2; r >= 0; --r) reduce_into(op, dt, all + (size_t)r * nb, acc, count);
    if (nb) memcpy(recvbuf, acc, nb);
  });
  return s.id;
}

int sched_reduce_scatter(Comm& c, const void* sendbuf, void* recvbuf, const std::vector<size_t>& counts,
                         MPI_Datatype dt, MPI_Op op) {
  const int p = (int)c.ranks.size();
  const size_t esz = type_info(dt).size;
  Sched s(c);
  std::vector<size_t> displ((size_t)p + 1, 0);
  for (int r = 0; r < p; ++r) displ[(size_t)r + 1] = displ[(size_t)r] + counts[(size_t)r];
  const size_t mycount = counts[(size_t)c.me], nb = mycount * esz;
  // the in-place form holds the input in recvbuf; copy it, the result overwrites its start
  const char* in;
  if (sendbuf == MPI_IN_PLACE) {
    char* copy = s.temp(displ[(size_t)p] * esz);
    if (displ[(size_t)p]) memcpy(copy, recvbuf, displ[(size_t)p] * esz);
    in = copy;
  } else {
    in = (const char*)sendbuf;
  }
  char* all = s.temp(nb * (size_t)p);
  if (nb) memcpy(all + (size_t)c.me * nb, in + displ[(size_t)c.me] * esz, nb);
  for (int r = 0; r < p; ++r)
    if (r != c.me) s.recv(all + (size_t)r * nb, nb, r);
  for (int r = 0; r < p; ++r)
    if (r != c.me) s.send(in + displ[(size_t)r] * esz, counts[(size_t)r] * esz, r);
  s.on_finish([=] {
    char* acc = all + (size_t)(p - 1) * nb;
    for (int r = p - 2; r >= 0; --r) reduce_into(op, dt, all + (size_t)r * nb, acc, mycount);
    if (nb) memcpy(recvbuf, acc, nb);
  });
  return s.id;
}

int sched_bcast(Comm& c, void* buf, size_t nb, int root) {
  const int p = (int)c.ranks.size();
  Sched s(c);
  if (c.me == root) {
    for (int r = 0; r < p; ++r)
      if (r != root) s.send(buf, nb, r);
  } else {
    s.recv(buf, nb, root);
  }
  return s.id;
}

int sched_barrier(Comm& c) {
  const int p = (int)c.ranks.size();
  Sched s(c);
  char* dummy = s.temp(1);
  for (int r = 0; r < p; ++r)
    if (r != c.me) s.recv(dummy, 0, r);
  for (int r = 0; r < p; ++r)
    if (r != c.me) s.send(dummy, 0, r);
  return s.id;
}

/** Gather-style movement: rank r's `sendbytes[r]` bytes end up at recvbuf + rdispl[r] on the receivers. */
int sched_gatherv(Comm& c, const void* sendbuf, size_t sendbytes, void* recvbuf, const std::vector<size_t>& rbytes,
                  const std::vector<size_t>& rdispl, int root /* -1: everyone receives */) {
  const int p = (int)c.ranks.size();
  Sched s(c);
  const bool receiver = root < 0 || c.me == root;
  const void* mine = sendbuf;
  if (sendbuf == MPI_IN_PLACE) mine = nullptr;  // own slice already in place
  if (receiver) {
    for (int r = 0; r < p; ++r) {
      if (r == c.me) {
        if (mine && rbytes[(size_t)r]) memmove((char*)recvbuf + rdispl[(size_t)r], mine, rbytes[(size_t)r]);
      } else {
        s.recv((char*)recvbuf + rdispl[(size_t)r], rbytes[(size_t)r], r);
      }
    }
  }
  const char* src = mine ? (const char*)mine : (const char*)recvbuf + rdispl[(size_t)c.me];
  const size_t nb = mine ? sendbytes : rbytes[(size_t)c.me];
  if (root < 0) {
    for (int r = 0; r < p; ++r)
      if (r != c.me) s.send(src, nb, r);
  } else if (c.me != root) {
    s.send(sendbuf, sendbytes, root);
  }
  return s.id;
}

int sched_scatterv(Comm& c, const void* sendbuf, const std::vector<size_t>& sbytes, const std::vector<size_t>& sdispl,
                   void* recvbuf, size_t recvbytes, int root) {
  const int p = (int)c.ranks.size();
  Sched s(c);
  if (c.me == root) {
    for (int r = 0; r < p; ++r) {
      if (r == root) {
        if (recvbuf != MPI_IN_PLACE && sbytes[(size_t)r])
          memmove(recvbuf, (const char*)sendbuf + sdispl[(size_t)r], sbytes[(size_t)r]);
      } else {
        s.send((const char*)sendbuf + sdispl[(size_t)r], sbytes[(size_t)r], r);
      }
    }
  } else {
    s.recv(recvbuf, recvbytes, root);
  }
  return s.id;
}

int sched_alltoallv(Comm& c, const void* sendbuf, const std::vector<size_t>& sbytes, const std::vector<size_t>& sdispl,
                    void* recvbuf, const std::vector<size_t>& rbytes, const std::vector<size_t>& rdispl) {
  const int p = (int)c.ranks.size();
  Sched s(c);
  const char* in = (const char*)sendbuf;
  const std::vector<size_t>* sb = &sbytes;
  const std::vector<size_t>* sd = &sdispl;
  if (sendbuf == MPI_IN_PLACE) {
    size_t extent = 0;
    for (int r = 0; r < p; ++r) extent = std::max(extent, rdispl[(size_t)r] + rbytes[(size_t)r]);
    char* copy = s.temp(extent);
    if (extent) memcpy(copy, recvbuf, extent);
    in = copy;
    sb = &rbytes;
    sd = &rdispl;
  }
  for (int r = 0; r < p; ++r) {
    if (r == c.me) {
      if ((*sb)[(size_t)r]) memmove((char*)recvbuf + rdispl[(size_t)r], in + (*sd)[(size_t)r], (*sb)[(size_t)r]);
    } else {
      s.recv((char*)recvbuf + rdispl[(size_t)r], rbytes[(size_t)r], r);
    }
  }
  for (int r = 0; r < p; ++r)
    if (r != c.me) s.send(in + (*sd)[(size_t)r], (*sb)[(size_t)r], r);
  return s.id;
}

std::vector<size_t> scaled(const int* v, int p, size_t esz) {
  std::vector<size_t> out((size_t)p);
  for (int i = 0; i < p; ++i) out[(size_t)i] = (size_t)v[i] * esz;
  return out;
}
std::vector<size_t> uniform(size_t each, int p) { return std::vector<size_t>((size_t)p, each); }
std::vector<size_t> strided(size_t each, int p) {
  std::vector<size_t> out((size_t)p);
  for (int i = 0; i < p; ++i) out[(size_t)i] = (size_t)i * each;
  return out;
}

int finish_blocking(std::unique_lock<std::recursive_mutex>& lk, int id, const char* what) {
  return wait_one(lk, id, nullptr, what);
}

// ------------------------------------------------------------------------------------------
// start-up
// ------------------------------------------------------------------------------------------
int env_int(const char* a, const char* b, int dflt) {
  const char* v = getenv(a);
  if (!v && b) v = getenv(b);
  return v ? atoi(v) : dflt;
}

sockaddr_un make_addr(const std::string& job, int rank, socklen_t* len) {
  sockaddr_un a{};
  a.sun_family = AF_UNIX;
  const std::string name = "mpishim-" + job + "-" + std::to_string(rank);
  a.sun_path[0] = '\0';
  memcpy(a.sun_path + 1, name.data(), std::min(name.size(), sizeof(a.sun_path) - 2));
  *len = (socklen_t)(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  return a;
}

void set_nonblocking(int fd) {
  const int fl = fcntl(fd, F_GETFL, 0);
  fcntl(fd, F_SETFL, fl | O_NONBLOCK);
  int sz = 8 << 20;
  setsockopt(fd, SOL_SOCKET, SO_SNDBUF, &sz, sizeof(sz));
  setsockopt(fd, SOL_SOCKET, SO_RCVBUF, &sz, sizeof(sz));
}

std::string connect_world() {
  g_rank = env_int("MPISHIM_RANK", "RANK", 0);
  g_size = env_int("MPISHIM_SIZE", "WORLD_SIZE", 1);
  if (g_size < 1 || g_rank < 0 || g_rank >= g_size) die("bad RANK / WORLD_SIZE");
  if (const char* t = getenv("MPISHIM_TIMEOUT_S")) g_timeout_s = atof(t);
  g_peers.assign((size_t)g_size, Peer());
  g_comms[1].used = true;
  g_comms[1].ctx = 2;
  g_comms[1].me = g_rank;
  g_comms[1].ranks.resize((size_t)g_size);
  for (int r = 0; r < g_size; ++r) g_comms[1].ranks[(size_t)r] = r;
  g_comms[2].used = true;
  g_comms[2].ctx = 4;
  g_comms[2].me = 0;
  g_comms[2].ranks = {g_rank};
  g_groups[1].used = true;  // MPI_GROUP_EMPTY
  std::string job;
  if (g_size == 1) return job;

  if (const char* j = getenv("MPISHIM_JOB")) job = j;
  else {
    const char* port = getenv("MASTER_PORT");
    job = std::to_string((long)getuid()) + "." + (port ? port : "0");
  }
  const int lfd = socket(AF_UNIX, SOCK_STREAM, 0);
  if (lfd < 0) die("socket");
  socklen_t alen;
  sockaddr_un a = make_addr(job, g_rank, &alen);
  if (bind(lfd, (sockaddr*)&a, alen) != 0) die("bind (is another job using the same MASTER_PORT / MPISHIM_JOB?)");
  if (listen(lfd, 64) != 0) die("listen");
  const double t0 = now_s();
  for (int r = 0; r < g_rank; ++r) {  // connect to the lower ranks
    for (;;) {
      const int fd = socket(AF_UNIX, SOCK_STREAM, 0);
      socklen_t blen;
      sockaddr_un b = make_addr(job, r, &blen);
      if (connect(fd, (sockaddr*)&b, blen) == 0) {
        const int32_t me = g_rank;
        if (::send(fd, &me, sizeof(me), MSG_NOSIGNAL) != (ssize_t)sizeof(me)) die("hello failed");
        g_peers[(size_t)r].fd = fd;
        break;
      }
      close(fd);
      if (now_s() - t0 > g_timeout_s) die("could not reach a lower rank (not started?)");
      usleep(2000);
    }
  }
  for (int k = g_rank + 1; k < g_size; ++k) {  // accept the higher ranks
    pollfd pf{lfd, POLLIN, 0};
    while (::poll(&pf, 1, 100) == 0)
      if (now_s() - t0 > g_timeout_s) die("a higher rank never connected");
    const int fd = accept(lfd, nullptr, nullptr);
    if (fd < 0) die("accept");
    int32_t who = -1;
    size_t got = 0;
    while (got < sizeof(who)) {
      const ssize_t n = ::recv(fd, (char*)&who + got, sizeof(who) - got, 0);
      if (n <= 0) die("hello not received");
      got += (size_t)n;
    }
    if (who <= g_rank || who >= g_size || g_peers[(size_t)who].fd >= 0) die("unexpected hello");
    g_peers[(size_t)who].fd = fd;
  }
  close(lfd);
  for (int r = 0; r < g_size; ++r)
    if (r != g_rank) set_nonblocking(g_peers[(size_t)r].fd);
  return job;
}

// ------------------------------------------------------------------------------------------
// MPI_Barrier(MPI_COMM_WORLD) on shared memory
// ------------------------------------------------------------------------------------------
// Benchmarks line the ranks up with MPI_Barrier(MPI_COMM_WORLD) before every timed call.  A barrier
// made of socket messages releases the ranks several microseconds apart, and that skew would be charged to
// the library under test; a single-node MPI does this on shared memory.  So does this one: one cache
// line in a POSIX shared-memory object, a counter and a generation number.  Other communicators, the
// non-blocking form and failures to set the object up use the message schedule.
struct ShmBarrier {
  std::atomic<uint32_t> count;
  std::atomic<uint32_t> generation;
};
ShmBarrier* g_shm_barrier = nullptr;

void setup_shm_barrier(const std::string& job) {
  if (g_size <= 1 || getenv("MPISHIM_NO_SHM")) return;
  const std::string name = "/mpishim-" + job;
  auto barrier_by_messages = [&] {
    std::unique_lock<std::recursive_mutex> lk(g_mu);
    const int id = sched_barrier(g_comms[1]);
    finish_blocking(lk, id, "MPI_Init");
  };
  int fd = -1;
  if (g_rank == 0) {
    shm_unlink(name.c_str());
    fd = shm_open(name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd >= 0 && ftruncate(fd, 4096) != 0) { close(fd); fd = -1; }
  }
  barrier_by_messages();  // the object exists (or rank 0 could not make it)
  if (g_rank != 0) fd = shm_open(name.c_str(), O_RDWR, 0600);
  void* mem = fd >= 0 ? mmap(nullptr, 4096, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0) : MAP_FAILED;
  if (fd >= 0) close(fd);
  // every rank has to have it, or nobody uses it
  int mine = mem != MAP_FAILED ? 1 : 0, everyone = 0;
  {
    std::unique_lock<std::recursive_mutex> lk(g_mu);
    const int id = sched_allreduce(g_comms[1], &mine, &everyone, 1, MPI_INT, MPI_MIN);
    finish_blocking(lk, id, "MPI_Init");
  }
  if (g_rank == 0) shm_unlink(name.c_str());  // the mappings keep it alive; nothing is left behind
  if (everyone) g_shm_barrier = (ShmBarrier*)mem;   // fresh pages of a new object are zero
  else if (mem != MAP_FAILED) munmap(mem, 4096);
}

/** true: done; false: not available (use the message schedule). */
bool shm_barrier_world() {
  ShmBarrier* b = g_shm_barrier;
  if (!b) return false;
  const uint32_t gen = b->generation.load(std::memory_order_acquire);
  if (b->count.fetch_add(1, std::memory_order_acq_rel) + 1 == (uint32_t)g_size) {
    b->count.store(0, std::memory_order_relaxed);
    b->generation.store(gen + 1, std::memory_order_release);
    return true;
  }
  const double t0 = now_s();
  for (unsigned spins = 0; b->generation.load(std::memory_order_acquire) == gen; ++spins) {
    if (spins > 20000) {
      sched_yield();
      if ((spins & 1023) == 0 && now_s() - t0 > g_timeout_s) die("MPI_Barrier: a rank never arrived");
    }
  }
  return true;
}

#define LOCK std::unique_lock<std::recursive_mutex> lk(g_mu)

}  // namespace

// ============================================================================================
// API
// ============================================================================================
extern "C" {

int MPI_Init_thread(int*, char***, int, int* provided) {
  LOCK;
  if (!g_initialized) {
    const std::string job = connect_world();
    g_initialized = true;
    lk.unlock();
    setup_shm_barrier(job);
    lk.lock();
  }
  if (provided) *provided = MPI_THREAD_MULTIPLE;
  return MPI_SUCCESS;
}
int MPI_Init(int* argc, char*** argv) { int p; return MPI_Init_thread(argc, argv, MPI_THREAD_MULTIPLE, &p); }
int MPI_Query_thread(int* provided) { *provided = MPI_THREAD_MULTIPLE; return MPI_SUCCESS; }
int MPI_Initialized(int* flag) { LOCK; *flag = g_initialized ? 1 : 0; return MPI_SUCCESS; }
int MPI_Finalized(int* flag) { LOCK; *flag = g_finalized ? 1 : 0; return MPI_SUCCESS; }
int MPI_Finalize(void) {
  LOCK;
  if (g_finalized) return MPI_SUCCESS;
  if (g_size > 1) {
    const int id = sched_barrier(comm_of(MPI_COMM_WORLD));
    finish_blocking(lk, id, "MPI_Finalize");
    for (auto& P : g_peers)
      if (P.fd >= 0) { close(P.fd); P.fd = -1; }
  }
  g_finalized = true;
  return MPI_SUCCESS;
}
int MPI_Abort(MPI_Comm, int errorcode) {
  fprintf(stderr, "[mpi_shim rank %d] MPI_Abort(%d)\n", g_rank, errorcode);
  fflush(stderr);
  _exit(errorcode ? errorcode : 1);
}
double MPI_Wtime(void) { return now_s(); }
int MPI_Get_processor_name(char* name, int* resultlen) {
  if (gethostname(name, MPI_MAX_PROCESSOR_NAME - 1) != 0) strcpy(name, "localhost");
  name[MPI_MAX_PROCESSOR_NAME - 1] = 0;
  *resultlen = (int)strlen(name);
  return MPI_SUCCESS;
}
int MPI_Get_version(int* version, int* subversion) { *version = MPI_VERSION; *subversion = MPI_SUBVERSION; return MPI_SUCCESS; }
int MPI_Get_library_version(char* version, int* resultlen) {
  strcpy(version, "mpi_shim 1.0 (single node, Unix sockets)");
  *resultlen = (int)strlen(version);
  return MPI_SUCCESS;
}
int MPI_Error_string(int errorcode, char* string, int* resultlen) {
  snprintf(string, MPI_MAX_ERROR_STRING, "mpi_shim error %d", errorcode);
  *resultlen = (int)strlen(string);
  return MPI_SUCCESS;
}
int MPI_Comm_set_errhandler(MPI_Comm, MPI_Errhandler) { return MPI_SUCCESS; }

// ---- communicators ---------------------------------------------------------------------------
int MPI_Comm_rank(MPI_Comm comm, int* rank) { LOCK; *rank = comm_of(comm).me; return MPI_SUCCESS; }
int MPI_Comm_size(MPI_Comm comm, int* size) { LOCK; *size = (int)comm_of(comm).ranks.size(); return MPI_SUCCESS; }

int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* newcomm) {
  LOCK;
  Comm& c = comm_of(comm);
  const int p = (int)c.ranks.size();
  struct Ent { int color, key, next_ctx, pad; };
  std::vector<Ent> all((size_t)p);
  Ent mine{color, key, g_next_ctx, 0};
  const int id = sched_gatherv(c, &mine, sizeof(Ent), all.data(), uniform(sizeof(Ent), p), strided(sizeof(Ent), p), -1);
  finish_blocking(lk, id, "MPI_Comm_split");
  Comm& c2 = comm_of(comm);  // the table may have been re-allocated
  int ctx = 0;
  for (const Ent& e : all) ctx = std::max(ctx, e.next_ctx);
  g_next_ctx = ctx + 2;
  if (color == MPI_UNDEFINED) { *newcomm = MPI_COMM_NULL; return MPI_SUCCESS; }
  std::vector<std::pair<std::pair<int, int>, int>> members;  // ((key, old rank), world rank)
  for (int r = 0; r < p; ++r)
    if (all[(size_t)r].color == color) members.push_back({{all[(size_t)r].key, r}, c2.ranks[(size_t)r]});
  std::sort(members.begin(), members.end());
  std::vector<int> ranks;
  for (auto& m : members) ranks.push_back(m.second);
  *newcomm = new_comm(ctx, std::move(ranks));
  return MPI_SUCCESS;
}
int MPI_Comm_dup(MPI_Comm comm, MPI_Comm* newcomm) {
  int me;
  MPI_Comm_rank(comm, &me);
  return MPI_Comm_split(comm, 0, me, newcomm);
}
int MPI_Comm_split_type(MPI_Comm comm, int, int key, MPI_Info, MPI_Comm* newcomm) {
  return MPI_Comm_split(comm, 0, key, newcomm);  // one node: everybody shares memory
}
int MPI_Comm_create(MPI_Comm comm, MPI_Group group, MPI_Comm* newcomm) {
  int color = MPI_UNDEFINED, key = 0;
  {
    LOCK;
    if (group <= 0 || (size_t)group >= g_groups.size() || !g_groups[(size_t)group].used) die("invalid group");
    const Group& g = g_groups[(size_t)group];
    for (size_t i = 0; i < g.ranks.size(); ++i)
      if (g.ranks[i] == g_rank) { color = 0; key = (int)i; }
  }
  return MPI_Comm_split(comm, color, key, newcomm);
}
int MPI_Comm_free(MPI_Comm* comm) {
  LOCK;
  if (*comm > 2) g_comms[(size_t)*comm] = Comm();
  *comm = MPI_COMM_NULL;
  return MPI_SUCCESS;
}
int MPI_Comm_get_attr(MPI_Comm, int keyval, void* attribute_val, int* flag) {
  if (keyval == MPI_TAG_UB) {
    *(int**)attribute_val = &g_tag_ub;
    *flag = 1;
  } else {
    *flag = 0;
  }
  return MPI_SUCCESS;
}
int MPI_Comm_compare(MPI_Comm a, MPI_Comm b, int* result) {
  LOCK;
  if (a == b) { *result = MPI_IDENT; return MPI_SUCCESS; }
  const Comm &x = comm_of(a), &y = comm_of(b);
  if (x.ranks == y.ranks) { *result = MPI_CONGRUENT; return MPI_SUCCESS; }
  std::vector<int> xs = x.ranks, ys = y.ranks;
  std::sort(xs.begin(), xs.end());
  std::sort(ys.begin(), ys.end());
  *result = xs == ys ? MPI_SIMILAR : MPI_UNEQUAL;
  return MPI_SUCCESS;
}
static MPI_Group new_group(std::vector<int> ranks) {
  size_t id = 2;
  while (id < g_groups.size() && g_groups[id].used) ++id;
  if (id == g_groups.size()) g_groups.emplace_back();
  Group& g = g_groups[id];
  g.used = true;
  g.ranks = std::move(ranks);
  g.me = MPI_UNDEFINED;
  for (size_t i = 0; i < g.ranks.size(); ++i)
    if (g.ranks[i] == g_rank) g.me = (int)i;
  return (MPI_Group)id;
}
int MPI_Comm_group(MPI_Comm comm, MPI_Group* group) { LOCK; *group = new_group(comm_of(comm).ranks); return MPI_SUCCESS; }
int MPI_Group_size(MPI_Group group, int* size) { LOCK; *size = (int)g_groups[(size_t)group].ranks.size(); return MPI_SUCCESS; }
int MPI_Group_rank(MPI_Group group, int* rank) { LOCK; *rank = g_groups[(size_t)group].me; return MPI_SUCCESS; }
int MPI_Group_incl(MPI_Group group, int n, const int ranks[], MPI_Group* newgroup) {
  LOCK;
  std::vector<int> out;
  for (int i = 0; i < n; ++i) out.push_back(g_groups[(size_t)group].ranks[(size_t)ranks[i]]);
  *newgroup = new_group(std::move(out));
  return MPI_SUCCESS;
}
int MPI_Group_translate_ranks(MPI_Group g1, int n, const int ranks1[], MPI_Group g2, int ranks2[]) {
  LOCK;
  const Group &a = g_groups[(size_t)g1], &b = g_groups[(size_t)g2];
  for (int i = 0; i < n; ++i) {
    ranks2[i] = MPI_UNDEFINED;
    if (ranks1[i] == MPI_PROC_NULL) { ranks2[i] = MPI_PROC_NULL; continue; }
    const int w = a.ranks[(size_t)ranks1[i]];
    for (size_t k = 0; k < b.ranks.size(); ++k)
      if (b.ranks[k] == w) ranks2[i] = (int)k;
  }
  return MPI_SUCCESS;
}
int MPI_Group_free(MPI_Group* group) {
  LOCK;
  if (*group > 1) g_groups[(size_t)*group] = Group();
  *group = MPI_GROUP_NULL;
  return MPI_SUCCESS;
}

// ---- datatypes, operators ----------------------------------------------------------------------
int MPI_Type_size(MPI_Datatype dt, int* size) { *size = (int)type_info(dt).size; return MPI_SUCCESS; }
int MPI_Get_count(const MPI_Status* status, MPI_Datatype dt, int* count) {
  *count = (int)((size_t)status->shim_bytes / type_info(dt).size);
  return MPI_SUCCESS;
}
int MPI_Op_create(MPI_User_function* fn, int, MPI_Op* op) {
  LOCK;
  size_t i = 0;
  while (i < g_ops.size() && g_ops[i].used) ++i;
  if (i == g_ops.size()) g_ops.emplace_back();
  g_ops[i].used = true;
  g_ops[i].fn = fn;
  *op = (MPI_Op)(16 + i);
  return MPI_SUCCESS;
}
int MPI_Op_free(MPI_Op* op) {
  LOCK;
  if (*op >= 16 && (size_t)(*op - 16) < g_ops.size()) g_ops[(size_t)(*op - 16)] = UserOp();
  *op = MPI_OP_NULL;
  return MPI_SUCCESS;
}

// ---- point to point ------------------------------------------------------------------------------
int MPI_Isend(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request* req) {
  LOCK;
  if (dest == MPI_PROC_NULL) { const int id = new_req(Req::kSend); g_reqs[(size_t)id].done = true; *req = id; return MPI_SUCCESS; }
  Comm& c = comm_of(comm);
  *req = post_send(buf, (size_t)count * type_info(dt).size, c.ranks[(size_t)dest], c.ctx, tag);
  return MPI_SUCCESS;
}
int MPI_Irecv(void* buf, int count, MPI_Datatype dt, int source, int tag, MPI_Comm comm, MPI_Request* req) {
  LOCK;
  if (source == MPI_PROC_NULL) {
    const int id = new_req(Req::kRecv);
    g_reqs[(size_t)id].done = true;
    g_reqs[(size_t)id].st.MPI_SOURCE = MPI_PROC_NULL;
    g_reqs[(size_t)id].st.MPI_TAG = MPI_ANY_TAG;
    *req = id;
    return MPI_SUCCESS;
  }
  if (source == MPI_ANY_SOURCE || tag == MPI_ANY_TAG) die("wildcard receives are not supported by mpi_shim");
  Comm& c = comm_of(comm);
  *req = post_recv(buf, (size_t)count * type_info(dt).size, c.ranks[(size_t)source], c.ctx, tag, source);
  return MPI_SUCCESS;
}
int MPI_Wait(MPI_Request* req, MPI_Status* status) {
  LOCK;
  if (*req == MPI_REQUEST_NULL) return MPI_SUCCESS;
  wait_one(lk, *req, status, "MPI_Wait");
  *req = MPI_REQUEST_NULL;
  return MPI_SUCCESS;
}
int MPI_Test(MPI_Request* req, int* flag, MPI_Status* status) {
  LOCK;
  if (*req == MPI_REQUEST_NULL) { *flag = 1; return MPI_SUCCESS; }
  progress();
  if (req_done(*req)) {
    if (status) *status = g_reqs[(size_t)*req].st;
    free_req(*req);
    *req = MPI_REQUEST_NULL;
    *flag = 1;
  } else {
    *flag = 0;
  }
  return MPI_SUCCESS;
}
int MPI_Waitall(int count, MPI_Request reqs[], MPI_Status statuses[]) {
  for (int i = 0; i < count; ++i) MPI_Wait(&reqs[i], statuses ? &statuses[i] : MPI_STATUS_IGNORE);
  return MPI_SUCCESS;
}
int MPI_Testall(int count, MPI_Request reqs[], int* flag, MPI_Status statuses[]) {
  LOCK;
  progress();
  for (int i = 0; i < count; ++i)
    if (reqs[i] != MPI_REQUEST_NULL && !req_done(reqs[i])) { *flag = 0; return MPI_SUCCESS; }
  for (int i = 0; i < count; ++i) {
    if (reqs[i] == MPI_REQUEST_NULL) continue;
    if (statuses) statuses[i] = g_reqs[(size_t)reqs[i]].st;
    free_req(reqs[i]);
    reqs[i] = MPI_REQUEST_NULL;
  }
  *flag = 1;
  return MPI_SUCCESS;
}
int MPI_Request_free(MPI_Request* req) {
  // the transfer still has to complete; it is simply waited for here
  return MPI_Wait(req, MPI_STATUS_IGNORE);
}
int MPI_Send(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm) {
  MPI_Request r;
  MPI_Isend(buf, count, dt, dest, tag, comm, &r);
  return MPI_Wait(&r, MPI_STATUS_IGNORE);
}
int MPI_Recv(void* buf, int count, MPI_Datatype dt, int source, int tag, MPI_Comm comm, MPI_Status* status) {
  MPI_Request r;
  MPI_Irecv(buf, count, dt, source, tag, comm, &r);
  return MPI_Wait(&r, status);
}
int MPI_Sendrecv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, int dest, int sendtag, void* recvbuf,
                 int recvcount, MPI_Datatype recvtype, int source, int recvtag, MPI_Comm comm, MPI_Status* status) {
  MPI_Request r[2];
  MPI_Irecv(recvbuf, recvcount, recvtype, source, recvtag, comm, &r[0]);
  MPI_Isend(sendbuf, sendcount, sendtype, dest, sendtag, comm, &r[1]);
  MPI_Wait(&r[0], status);
  return MPI_Wait(&r[1], MPI_STATUS_IGNORE);
}
int MPI_Sendrecv_replace(void* buf, int count, MPI_Datatype dt, int dest, int sendtag, int source, int recvtag,
                         MPI_Comm comm, MPI_Status* status) {
  const size_t nb = (size_t)count * type_info(dt).size;
  std::vector<char> copy((const char*)buf, (const char*)buf + nb);
  return MPI_Sendrecv(copy.data(), count, dt, dest, sendtag, buf, count, dt, source, recvtag, comm, status);
}
int MPI_Isendrecv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, int dest, int sendtag, void* recvbuf,
                  int recvcount, MPI_Datatype recvtype, int source, int recvtag, MPI_Comm comm, MPI_Request* req) {
  LOCK;
  MPI_Request a, b;
  MPI_Irecv(recvbuf, recvcount, recvtype, source, recvtag, comm, &a);
  MPI_Isend(sendbuf, sendcount, sendtype, dest, sendtag, comm, &b);
  const int id = new_req(Req::kColl);
  g_reqs[(size_t)id].children = {a, b};
  *req = id;
  return MPI_SUCCESS;
}

// ---- collectives -----------------------------------------------------------------------------------
#define COLL_BEGIN LOCK; Comm& c = comm_of(comm); const int p = (int)c.ranks.size(); (void)p
#define COLL_RETURN(idexpr, name)                 \
  do {                                            \
    const int id__ = (idexpr);                    \
    if (req) { *req = id__; return MPI_SUCCESS; } \
    return finish_blocking(lk, id__, name);       \
  } while (0)

static int do_barrier(MPI_Comm comm, MPI_Request* req) { COLL_BEGIN; COLL_RETURN(sched_barrier(c), "MPI_Barrier"); }
static int do_bcast(void* buf, int count, MPI_Datatype dt, int root, MPI_Comm comm, MPI_Request* req) {
  COLL_BEGIN;
  COLL_RETURN(sched_bcast(c, buf, (size_t)count * type_info(dt).size, root), "MPI_Bcast");
}
static int do_reduce(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm, MPI_Request* req) {
  COLL_BEGIN;
  COLL_RETURN(sched_reduce(c, s, r, (size_t)count, dt, op, root), "MPI_Reduce");
}
static int do_allreduce(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm, MPI_Request* req) {
  COLL_BEGIN;
  COLL_RETURN(sched_allreduce(c, s, r, (size_t)count, dt, op), "MPI_Allreduce");
}
static int do_reduce_scatter(const void* s, void* r, const int counts[], int block, MPI_Datatype dt, MPI_Op op,
                             MPI_Comm comm, MPI_Request* req) {
  COLL_BEGIN;
  std::vector<size_t> cnt((size_t)p);
  for (int i = 0; i < p; ++i) cnt[(size_t)i] = counts ? (size_t)counts[i] : (size_t)block;
  COLL_RETURN(sched_reduce_scatter(c, s, r, cnt, dt, op), "MPI_Reduce_scatter");
}
static int do_allgatherv(const void* s, int scount, MPI_Datatype st, void* r, const int rcounts[], const int displs[],
                         int rcount, MPI_Datatype rt, int root, MPI_Comm comm, MPI_Request* req) {
  COLL_BEGIN;
  std::vector<size_t> rb, rd;
  if (root < 0 || c.me == root) {  // the receive arguments are significant on receivers only
    const size_t resz = type_info(rt).size;
    rb = rcounts ? scaled(rcounts, p, resz) : uniform((size_t)rcount * resz, p);
    rd = displs ? scaled(displs, p, resz) : strided((size_t)rcount * resz, p);
  }
  const size_t sb = s == MPI_IN_PLACE ? 0 : (size_t)scount * type_info(st).size;
  COLL_RETURN(sched_gatherv(c, s, sb, r, rb, rd, root), "MPI_(All)gather(v)");
}
static int do_scatterv(const void* s, const int scounts[], const int displs[], int scount, MPI_Datatype st, void* r,
                       int rcount, MPI_Datatype rt, int root, MPI_Comm comm, MPI_Request* req) {
  COLL_BEGIN;
  std::vector<size_t> sb, sd;
  if (c.me == root) {
    const size_t sesz = type_info(st).size;
    sb = scounts ? scaled(scounts, p, sesz) : uniform((size_t)scount * sesz, p);
    sd = displs ? scaled(displs, p, sesz) : strided((size_t)scount * sesz, p);
  }
  const size_t rb = r == MPI_IN_PLACE ? 0 : (size_t)rcount * type_info(rt).size;
  COLL_RETURN(sched_scatterv(c, s, sb, sd, r, rb, root), "MPI_Scatter(v)");
}
static int do_alltoallv(const void* s, const int scounts[], const int sdispls[], int scount, MPI_Datatype st, void* r,
                        const int rcounts[], const int rdispls[], int rcount, MPI_Datatype rt, MPI_Comm comm,
                        MPI_Request* req) {
  COLL_BEGIN;
  const size_t resz = type_info(rt).size;
  std::vector<size_t> rb = rcounts ? scaled(rcounts, p, resz) : uniform((size_t)rcount * resz, p);
  std::vector<size_t> rd = rdispls ? scaled(rdispls, p, resz) : strided((size_t)rcount * resz, p);
  std::vector<size_t> sb, sd;
  if (s != MPI_IN_PLACE) {
    const size_t sesz = type_info(st).size;
    sb = scounts ? scaled(scounts, p, sesz) : uniform((size_t)scount * sesz, p);
    sd = sdispls ? scaled(sdispls, p, sesz) : strided((size_t)scount * sesz, p);
  }
  COLL_RETURN(sched_alltoallv(c, s, sb, sd, r, rb, rd), "MPI_Alltoall(v)");
}

int MPI_Barrier(MPI_Comm comm) {
  if (comm == MPI_COMM_WORLD && shm_barrier_world()) return MPI_SUCCESS;
  return do_barrier(comm, nullptr);
}
int MPI_Ibarrier(MPI_Comm comm, MPI_Request* req) { return do_barrier(comm, req); }
int MPI_Bcast(void* buf, int count, MPI_Datatype dt, int root, MPI_Comm comm) { return do_bcast(buf, count, dt, root, comm, nullptr); }
int MPI_Ibcast(void* buf, int count, MPI_Datatype dt, int root, MPI_Comm comm, MPI_Request* req) { return do_bcast(buf, count, dt, root, comm, req); }
int MPI_Reduce(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm) { return do_reduce(s, r, count, dt, op, root, comm, nullptr); }
int MPI_Ireduce(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm, MPI_Request* req) { return do_reduce(s, r, count, dt, op, root, comm, req); }
int MPI_Allreduce(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) { return do_allreduce(s, r, count, dt, op, comm, nullptr); }
int MPI_Iallreduce(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm, MPI_Request* req) { return do_allreduce(s, r, count, dt, op, comm, req); }
int MPI_Reduce_scatter(const void* s, void* r, const int counts[], MPI_Datatype dt, MPI_Op op, MPI_Comm comm) { return do_reduce_scatter(s, r, counts, 0, dt, op, comm, nullptr); }
int MPI_Ireduce_scatter(const void* s, void* r, const int counts[], MPI_Datatype dt, MPI_Op op, MPI_Comm comm, MPI_Request* req) { return do_reduce_scatter(s, r, counts, 0, dt, op, comm, req); }
int MPI_Reduce_scatter_block(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm) { return do_reduce_scatter(s, r, nullptr, count, dt, op, comm, nullptr); }
int MPI_Ireduce_scatter_block(const void* s, void* r, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm, MPI_Request* req) { return do_reduce_scatter(s, r, nullptr, count, dt, op, comm, req); }
int MPI_Allgather(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, MPI_Comm comm) { return do_allgatherv(s, sc, st, r, nullptr, nullptr, rc, rt, -1, comm, nullptr); }
int MPI_Iallgather(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, MPI_Comm comm, MPI_Request* req) { return do_allgatherv(s, sc, st, r, nullptr, nullptr, rc, rt, -1, comm, req); }
int MPI_Allgatherv(const void* s, int sc, MPI_Datatype st, void* r, const int rcs[], const int ds[], MPI_Datatype rt, MPI_Comm comm) { return do_allgatherv(s, sc, st, r, rcs, ds, 0, rt, -1, comm, nullptr); }
int MPI_Iallgatherv(const void* s, int sc, MPI_Datatype st, void* r, const int rcs[], const int ds[], MPI_Datatype rt, MPI_Comm comm, MPI_Request* req) { return do_allgatherv(s, sc, st, r, rcs, ds, 0, rt, -1, comm, req); }
int MPI_Gather(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, int root, MPI_Comm comm) { return do_allgatherv(s, sc, st, r, nullptr, nullptr, rc, rt, root, comm, nullptr); }
int MPI_Igather(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, int root, MPI_Comm comm, MPI_Request* req) { return do_allgatherv(s, sc, st, r, nullptr, nullptr, rc, rt, root, comm, req); }
int MPI_Gatherv(const void* s, int sc, MPI_Datatype st, void* r, const int rcs[], const int ds[], MPI_Datatype rt, int root, MPI_Comm comm) { return do_allgatherv(s, sc, st, r, rcs, ds, 0, rt, root, comm, nullptr); }
int MPI_Igatherv(const void* s, int sc, MPI_Datatype st, void* r, const int rcs[], const int ds[], MPI_Datatype rt, int root, MPI_Comm comm, MPI_Request* req) { return do_allgatherv(s, sc, st, r, rcs, ds, 0, rt, root, comm, req); }
int MPI_Scatter(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, int root, MPI_Comm comm) { return do_scatterv(s, nullptr, nullptr, sc, st, r, rc, rt, root, comm, nullptr); }
int MPI_Iscatter(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, int root, MPI_Comm comm, MPI_Request* req) { return do_scatterv(s, nullptr, nullptr, sc, st, r, rc, rt, root, comm, req); }
int MPI_Scatterv(const void* s, const int scs[], const int ds[], MPI_Datatype st, void* r, int rc, MPI_Datatype rt, int root, MPI_Comm comm) { return do_scatterv(s, scs, ds, 0, st, r, rc, rt, root, comm, nullptr); }
int MPI_Iscatterv(const void* s, const int scs[], const int ds[], MPI_Datatype st, void* r, int rc, MPI_Datatype rt, int root, MPI_Comm comm, MPI_Request* req) { return do_scatterv(s, scs, ds, 0, st, r, rc, rt, root, comm, req); }
int MPI_Alltoall(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, MPI_Comm comm) { return do_alltoallv(s, nullptr, nullptr, sc, st, r, nullptr, nullptr, rc, rt, comm, nullptr); }
int MPI_Ialltoall(const void* s, int sc, MPI_Datatype st, void* r, int rc, MPI_Datatype rt, MPI_Comm comm, MPI_Request* req) { return do_alltoallv(s, nullptr, nullptr, sc, st, r, nullptr, nullptr, rc, rt, comm, req); }
int MPI_Alltoallv(const void* s, const int scs[], const int sds[], MPI_Datatype st, void* r, const int rcs[], const int rds[], MPI_Datatype rt, MPI_Comm comm) { return do_alltoallv(s, scs, sds, 0, st, r, rcs, rds, 0, rt, comm, nullptr); }
int MPI_Ialltoallv(const void* s, const int scs[], const int sds[], MPI_Datatype st, void* r, const int rcs[], const int rds[], MPI_Datatype rt, MPI_Comm comm, MPI_Request* req) { return do_alltoallv(s, scs, sds, 0, st, r, rcs, rds, 0, rt, comm, req); }

}  // extern "C"
