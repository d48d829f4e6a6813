// Private to the host backend: the socket data plane of a communicator whose
// ranks are on more than one node.
//
// The reference reaches other nodes through MPI (src/mpi_impl.cpp,
// include/aluminum/mpi/*.hpp).  Here every such communicator owns two TCP
// connections per pair of ranks - one carries collectives, one point-to-point
// traffic - and all transfers are non-blocking, driven by the progress engine
// or, for blocking calls, by the calling thread.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "al/bootstrap.hpp"

namespace Al {
namespace internal {
namespace host {

/** Precedes every message; lets the receiver detect mismatched calls instead of misreading bytes. */
struct NetHeader {
  uint32_t magic = 0;
  uint32_t round = 0;
  uint64_t seq = 0;
  uint64_t bytes = 0;
};

enum NetChannel { kNetCollectives = 0, kNetPointToPoint = 1 };

/** The sockets of one communicator: fd(channel, peer), non-blocking, TCP_NODELAY. */
class NetMesh {
 public:
  /** Collective over the members of `g`. */
  explicit NetMesh(const Group& g);
  ~NetMesh();
  NetMesh(const NetMesh&) = delete;
  NetMesh& operator=(const NetMesh&) = delete;
  int fd(int channel, int peer) const { return fds_[channel][(size_t)peer]; }
  int size() const { return p_; }
  int rank() const { return me_; }
  /** Shut every connection down (both directions): the peers' pending reads end with "connection closed". */
  void shutdown_all() const;

 private:
  int p_ = 1, me_ = 0;
  std::vector<int> fds_[2];
};

/** One message of a round. */
struct NetXfer {
  int peer = -1;
  bool is_send = false;
  char* buf = nullptr;
  size_t bytes = 0;
  NetHeader hdr;   ///< what is sent, or what a receive expects
  NetHeader got;   ///< what a receive actually read
  size_t hdr_done = 0, done = 0;
  bool complete() const { return hdr_done == sizeof(NetHeader) && done == bytes; }
};

/**
 * A set of messages that progress together without ever blocking.  Messages to
 * (from) the same peer move in the order they were added.
 */
class NetRound {
 public:
  enum Status { pending, done, error };
  void send(int peer, const void* buf, size_t bytes);
  void recv(int peer, void* buf, size_t bytes);
  /** Stamps the headers; call once, after the last send()/recv(). */
  void seal(uint64_t seq, uint32_t round);
  /** Moves whatever the sockets accept or hold right now. */
  Status progress(const NetMesh& mesh, int channel, bool* moved, std::string* err);
  /** Peer of the first incomplete message (for time-out reports), -1 if none. */
  int waiting_for() const;
  bool empty() const { return xfers_.empty(); }

 private:
  std::vector<NetXfer> xfers_;
  std::vector<char> busy_;
};

}  // namespace host
}  // namespace internal
}  // namespace Al
