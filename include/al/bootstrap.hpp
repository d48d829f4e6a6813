/**
 * @file bootstrap.hpp
 * Host control plane: rank discovery from the launcher's environment and a
 * full mesh of stream sockets between the ranks - Unix-domain sockets between
 * ranks of one node (they can pass file descriptors), TCP between nodes - used
 * to exchange memory handles, shared-memory names, addresses and communicator
 * ids.
 *
 * This takes the place of MPI in the reference, where every communicator
 * duplicates an MPI_Comm, derives the node-local communicator with
 * MPI_Comm_split_type and broadcasts the NCCL id over MPI
 * (include/aluminum/mpi_comm_and_stream_wrapper.hpp:46-129,
 * src/nccl_impl.cpp:46-60, src/mpi_impl.cpp:148-205).
 *
 * Transports (AL_TRANSPORT = auto | unix | tcp, default auto):
 *   unix  every rank is on this host; ranks find each other through abstract
 *         socket names derived from the job key.
 *   tcp   ranks may be on several hosts: rank 0 listens on
 *         MASTER_ADDR:AL_MASTER_PORT (default MASTER_PORT + 1), collects every
 *         rank's node name, address and listening port and hands the table to
 *         everyone; pairs on the same node still connect through Unix sockets.
 *         AL_MASTER_FD (set by alrun --nodes) passes rank 0 a socket that is
 *         already listening on that port.
 *   auto  tcp when MASTER_ADDR is set and the launcher reports more ranks than
 *         local ranks (LOCAL_WORLD_SIZE < WORLD_SIZE, SLURM_NNODES > 1,
 *         AL_NNODES > 1), else unix.
 * A rank's node is AL_NODE_ID when set (tests use it to model several nodes on
 * one machine), else its host name.
 *
 * Launcher variables understood (first match wins), mirroring the set the
 * reference's test helpers read (test/test_utils.hpp:463-530):
 *   AL_RANK/AL_WORLD_SIZE/AL_LOCAL_RANK, RANK/WORLD_SIZE/LOCAL_RANK (torchrun),
 *   OMPI_COMM_WORLD_*, PMI_RANK/PMI_SIZE, SLURM_PROCID/SLURM_NTASKS/SLURM_LOCALID,
 *   FLUX_TASK_RANK/FLUX_JOB_SIZE.
 * The rendezvous key is AL_JOB_KEY, else MASTER_ADDR:MASTER_PORT, else the
 * launcher's job id; ranks with the same key find each other.
 */
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "al/base.hpp"

namespace Al {
namespace internal {

/** Test hooks that make the control plane misbehave on the host only. */
struct BootstrapFaults {
  int drop_send_to = -1;      ///< silently drop the next message addressed to this world rank
  int drops_left = 0;
  double recv_timeout_s = -1; ///< override of the receive time-out (<0: use AL_BOOTSTRAP_TIMEOUT_S, default 120)
};

class World {
 public:
  /** Discover rank/size from the environment and connect the mesh. */
  static std::unique_ptr<World> from_env();
  /** Explicit construction (used by tests that fork ranks themselves). */
  static std::unique_ptr<World> connect(int rank, int size, int local_rank, const std::string& job_key);
  /** Multi-host construction: rendezvous at master_addr:master_port (see the file comment). */
  static std::unique_ptr<World> connect_tcp(int rank, int size, int local_rank_hint, const std::string& job_key,
                                            const std::string& master_addr, int master_port,
                                            const std::string& node_id);
  ~World();

  int rank() const { return rank_; }
  int size() const { return size_; }
  int local_rank() const { return local_rank_; }
  int local_size() const { return local_size_; }
  const std::string& job_key() const { return key_; }
  /** Node name of a rank; ranks with equal names share memory and can pass descriptors. */
  const std::string& node_of(int rank) const { return nodes_.at((size_t)rank); }
  bool same_node(int rank) const { return nodes_.at((size_t)rank) == nodes_.at((size_t)rank_); }
  /** Number of distinct nodes. */
  int num_nodes() const { return num_nodes_; }
  /** Position of a rank's node among the distinct nodes, numbered in order of their lowest rank. */
  int node_index(int rank) const;
  /** IP address (text) under which `rank` is reachable from other nodes. */
  const std::string& address_of(int rank) const { return addrs_.at((size_t)rank); }

  void send(int peer, const void* buf, size_t bytes);
  void recv(int peer, void* buf, size_t bytes);
  /** Pass an open file descriptor to `peer` (SCM_RIGHTS). */
  void send_fd(int peer, int fd);
  int recv_fd(int peer);

  /**
   * False once `peer`'s end of the control connection is closed: the process
   * has exited (or finalised the library) and will never take part in anything
   * again.  Non-blocking; safe to call from any thread.
   */
  bool peer_alive(int peer) const;

  /** Serialises whole collectives issued by different threads. */
  std::mutex& collective_mutex() { return coll_mu_; }
  BootstrapFaults faults;

 private:
  World() = default;
  int rank_ = 0, size_ = 1, local_rank_ = 0, local_size_ = 1;
  std::string key_;
  std::vector<int> socks_;  // socks_[peer], -1 for self
  std::vector<std::string> nodes_, addrs_;
  int num_nodes_ = 1;
  int listen_fd_ = -1, tcp_listen_fd_ = -1;
  void mesh(const std::vector<int>& tcp_ports, double tmo);
  std::mutex coll_mu_;
};

/** A TCP listening socket on an ephemeral port (returned in *port). */
int bootstrap_tcp_listen(int* port);
/** Connects to ip:port with TCP_NODELAY set, retrying for timeout_s seconds; -1 when the time is up. */
int bootstrap_tcp_connect(const std::string& ip, int port, double timeout_s);

/**
 * An ordered subset of the world; the unit on which communicators are built.
 * All methods are collective over the members and must be called in the same
 * order by each of them.
 */
class Group {
 public:
  Group() = default;
  Group(World* w, std::vector<int> members);
  static Group world_group(World* w);

  World* world() const { return world_; }
  int rank() const { return me_; }
  int size() const { return (int)members_.size(); }
  int world_rank_of(int r) const { return members_[(size_t)r]; }
  const std::vector<int>& members() const { return members_; }
  /** True when every member is on this rank's node (shared memory and descriptor passing work). */
  bool single_node() const;

  void allgather(const void* in, void* out, size_t bytes_per_rank) const;
  void bcast(void* buf, size_t bytes, int root) const;
  void barrier() const;
  /** Every rank contributes one descriptor and receives everyone's (its own slot holds a dup). */
  std::vector<int> allgather_fd(int fd) const;
  /** MPI_Comm_split semantics: ranks with equal color form a group ordered by (key, old rank). */
  Group split(int color, int key) const;
  /** A number that is identical on every member and unique per call within the process set. */
  uint64_t agree_on_id() const;

 private:
  World* world_ = nullptr;
  std::vector<int> members_;
  int me_ = 0;
};

}  // namespace internal
}  // namespace Al
