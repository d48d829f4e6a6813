/**
 * @file communicator.hpp
 * Communicator of the device backend and its type-erased operations.
 *
 * Role: the reference's NCCLCommunicator (include/aluminum/nccl_impl.hpp:110-155,
 * src/nccl_impl.cpp:43-79) - an ordered set of ranks plus the CUDA stream on
 * which "blocking" operations are enqueued.  Instead of an ncclComm_t it owns
 * a symmetric workspace (staging halves, epoch flags, mailboxes; multicast
 * alias when the GPUs support NVLS) and a pinned status record that kernels
 * fill when a bounded wait runs out.
 *
 * Semantics kept from the reference: operations are stream-ordered, the host
 * never blocks; non-blocking operations run on a pooled high-priority stream
 * bracketed by events (nccl_impl.hpp:902-940); communicators are move-only
 * and `copy(stream)` makes an independent communicator over the same ranks.
 * Operations of one communicator are serialised in issue order even when they
 * were enqueued on different streams.
 */
#pragma once
#include <memory>
#include <string>
#include <vector>

#include "al/bootstrap.hpp"
#include "al/cuda/cuda.hpp"
#include "al/device/params.hpp"
#include "al/device/symmem.hpp"

namespace Al {

namespace internal {
namespace device {

/** Algorithm selector of the device allreduce (the reference's `algo` argument, made real). */
enum class AllreduceAlgo : int { automatic = 0, one_shot, two_shot, nvls };

/** Arguments of one collective for one local rank. */
struct RankArgs {
  const void* send = nullptr;
  void* recv = nullptr;
  std::vector<size_t> send_counts, send_displs, recv_counts, recv_displs;  // vector forms only
};

struct CollDesc {
  DevColl kind = DevColl::barrier;
  DType in = DType::u8, wire = DType::u8, out = DType::u8;
  ReductionOperator op = ReductionOperator::sum;
  int root = 0;
  size_t count = 0;       ///< uniform count in elements
  bool vector = false;
  double scale = 1.0;     ///< extra factor applied to reduction results (on top of 1/p for avg)
  AllreduceAlgo algo = AllreduceAlgo::automatic;
  int ctas = 0;           ///< 0 = choose from the tuning table
};

struct P2PDesc {
  bool is_send = false;
  int peer = -1;
  const void* sbuf = nullptr;
  void* rbuf = nullptr;
  size_t bytes = 0;
  int owner = -1;         ///< emulation only: local rank issuing the transfer (-1 = this rank)
};

/** Counters readable from C++ and Python (observability). */
struct CommStats {
  uint64_t ops = 0, bytes = 0, kernels = 0, timeouts = 0;
  uint64_t ar_one_shot = 0, ar_two_shot = 0, ar_nvls = 0, ar_nvls_zero_copy = 0;
  uint64_t bulk_pipeline = 0;   ///< operations run by the bulk-copy pipeline kernel
  uint64_t direct = 0;          ///< allgather / alltoall stored straight into symmetric receive buffers
};

}  // namespace device
}  // namespace internal

class DeviceCommunicator {
 public:
  /** World communicator on the default stream (collective). */
  DeviceCommunicator();
  explicit DeviceCommunicator(cudaStream_t stream);
  DeviceCommunicator(const internal::Group& group, cudaStream_t stream);
  /** Communicator over the listed world ranks, in that order; collective over those ranks only. */
  static DeviceCommunicator from_ranks(const std::vector<int>& world_ranks, cudaStream_t stream = nullptr);
  /** All `p` ranks in this process on the current device (kernel tests on one GPU). */
  static DeviceCommunicator emulated(int p, cudaStream_t stream);
  ~DeviceCommunicator();
  DeviceCommunicator(DeviceCommunicator&&) noexcept;
  DeviceCommunicator& operator=(DeviceCommunicator&&) noexcept;
  DeviceCommunicator(const DeviceCommunicator&) = delete;
  DeviceCommunicator& operator=(const DeviceCommunicator&) = delete;

  DeviceCommunicator copy(cudaStream_t stream = nullptr) const;
  DeviceCommunicator split(int color, int key, cudaStream_t stream = nullptr) const;

  int rank() const;
  int size() const;
  int local_rank() const { return rank(); }
  int local_size() const { return size(); }
  cudaStream_t get_stream() const { return stream_; }
  const internal::Group& group() const { return group_; }
  bool is_emulated() const;
  bool has_multicast() const;
  const char* memory_backing() const;

  /**
   * Enqueue a collective on `stream`.  `ranks` has one entry per local rank
   * (exactly one outside emulation).
   */
  void collective(const internal::device::CollDesc& d, const std::vector<internal::device::RankArgs>& ranks,
                  cudaStream_t stream);
  /** Enqueue point-to-point transfers that progress together. */
  void p2p(const std::vector<internal::device::P2PDesc>& items, cudaStream_t stream);

  /** Collective allocation of symmetric memory (multicast-bound when possible). Returns this rank's pointer. */
  void* symm_alloc(size_t bytes);
  void symm_free(void* ptr);
  /** The symmetric block containing `ptr`, or nullptr. */
  const internal::device::SymmBlock* find_symm(const void* ptr, size_t bytes, size_t* offset) const;

  /** Position of the symmetric block containing `ptr` in allocation order (-1 if none); identical on every rank. */
  int symm_index(const void* ptr) const;
  /** Address, in this process, of rank `peer`'s copy of symmetric block `index` at byte `offset`. */
  void* symm_peer_ptr(int index, int peer, size_t offset) const;
  uint64_t wait_timeout_ns() const;

  /** Throws al_exception if a kernel of this communicator reported a failure. */
  void check_status() const;
  /**
   * Mark the communicator unusable on this rank: every later call throws.
   * Kernels already enqueued still end by themselves (their waits are
   * bounded).  Recovery is abort() on the surviving ranks followed by a new
   * communicator; the reference has no equivalent.
   */
  void abort(const std::string& why = "aborted by the caller");
  /** Non-throwing form: copy of the status record. */
  internal::device::DeviceStatus status() const;
  internal::device::CommStats stats() const;
  /** Bound of device-side waits for subsequent launches (milliseconds). */
  void set_wait_timeout_ms(double ms);
  /** Workspace description (used by RMA and halo code). */
  const internal::device::Workspace& workspace() const;
  uint64_t next_halo_epoch();

  struct Impl;
  Impl* impl() const { return impl_.get(); }

 private:
  DeviceCommunicator(std::shared_ptr<Impl> impl, const internal::Group& g, cudaStream_t s);
  internal::Group group_;
  cudaStream_t stream_ = nullptr;
  std::shared_ptr<Impl> impl_;
};

}  // namespace Al
