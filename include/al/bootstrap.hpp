/**
 * @file bootstrap.hpp
 * Host control plane: rank discovery from the launcher's environment and a
 * full mesh of Unix-domain sockets between the ranks of one node, used to
 * exchange memory handles (including file descriptors), shared-memory names
 * and communicator ids.
 *
 * This takes the place of MPI in the reference, where every communicator
 * duplicates an MPI_Comm, derives the node-local communicator with
 * MPI_Comm_split_type and broadcasts the NCCL id over MPI
 * (include/aluminum/mpi_comm_and_stream_wrapper.hpp:46-129,
 * src/nccl_impl.cpp:46-60, src/mpi_impl.cpp:148-205).  Scope: the ranks of one
 * NVLink domain / one host.
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
  ~World();

  int rank() const { return rank_; }
  int size() const { return size_; }
  int local_rank() const { return local_rank_; }
  int local_size() const { return local_size_; }
  const std::string& job_key() const { return key_; }

  void send(int peer, const void* buf, size_t bytes);
  void recv(int peer, void* buf, size_t bytes);
  /** Pass an open file descriptor to `peer` (SCM_RIGHTS). */
  void send_fd(int peer, int fd);
  int recv_fd(int peer);

  /** Serialises whole collectives issued by different threads. */
  std::mutex& collective_mutex() { return coll_mu_; }
  BootstrapFaults faults;

 private:
  World() = default;
  int rank_ = 0, size_ = 1, local_rank_ = 0, local_size_ = 1;
  std::string key_;
  std::vector<int> socks_;  // socks_[peer], -1 for self
  int listen_fd_ = -1;
  std::mutex coll_mu_;
};

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
