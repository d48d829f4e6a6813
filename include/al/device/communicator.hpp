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
enum class AllreduceAlgo : int { automatic = 0, one_shot, two_shot, nvls, ll };

/**
 * Data path of the other collectives (their `algo` argument):
 *   staged     through the communicator's staging area (any buffer; large uniform messages are
 *              pipelined, optionally by the bulk-copy engine - see the tuning table);
 *   window     reduce_scatter / allgather / alltoall / bcast straight on registered buffers
 *              (RegisterMemory or symm_alloc); an error if this rank's buffer is not registered.
 *   ll         small reduce_scatter / allgather / alltoall as low-latency packets (kernels/ll.cu);
 *              an error if the message does not fit (kLLPayloadBytes from one rank to another).
 *   nvls       reduce_scatter of private buffers reduced by the switch: copy into the multicast-bound staging,
 *              multimem.ld_reduce of the own slice straight into the receive buffer (kernels/nvls.cu); an error
 *              without multicast, on two ranks, or for types / operators the switch does not reduce.
 * `automatic` takes packets up to tuning().ll_max_bytes, the window path for registered buffers from
 * tuning().window_min_bytes on, the switch for large reduce_scatters (rs_nvls_min_bytes), staging otherwise.
 * AllreduceAlgo::ll is the same for allreduce.
 */
enum class CollPath : int { automatic = 0, staged, window, ll, nvls };

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
  CollPath path = CollPath::automatic;
  int ctas = 0;           ///< 0 = choose from the tuning table
};

/** Arguments of a row exchange for one local rank (see RowsParams in al/device/params.hpp). */
struct RowArgs {
  const void* send = nullptr;
  void* recv = nullptr;
  const long long* send_idx = nullptr;   ///< device memory, or nullptr
  const long long* recv_idx = nullptr;
  std::vector<size_t> send_rows, send_first, send_peer_off, recv_rows, recv_first, recv_peer_off;  ///< one entry per rank
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
  uint64_t window = 0;          ///< operations that ran straight on registered buffers (window kernels)
  uint64_t rs_nvls = 0;         ///< reduce_scatters of private buffers that the switch reduced (staged NVLS)
  uint64_t ll = 0;              ///< operations that ran as low-latency packets
  uint64_t rows = 0;            ///< row exchanges (alltoall with fused pack / unpack)
};

}  // namespace device
}  // namespace internal

/**
 * Makes a communicator's device current for the calling thread for the duration of a call and restores the
 * previous one.  A thread that was never told which device to use (cudaSetDevice is per thread) would
 * otherwise launch on device 0 into streams of another device.
 */
class ScopedDevice {
 public:
  explicit ScopedDevice(int device) {
    if (cudaGetDevice(&prev_) == cudaSuccess && prev_ != device && device >= 0) {
      switched_ = cudaSetDevice(device) == cudaSuccess;
    }
  }
  ~ScopedDevice() {
    if (switched_) (void)cudaSetDevice(prev_);
  }
  ScopedDevice(const ScopedDevice&) = delete;
  ScopedDevice& operator=(const ScopedDevice&) = delete;

 private:
  int prev_ = -1;
  bool switched_ = false;
};

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
  /** The CUDA device the communicator was created on (its workspace, streams and kernels live there). */
  int device() const;
  bool has_multicast() const;
  const char* memory_backing() const;

  /**
   * Enqueue a collective on `stream`.  `ranks` has one entry per local rank
   * (exactly one outside emulation).
   */
  void collective(const internal::device::CollDesc& d, const std::vector<internal::device::RankArgs>& ranks,
                  cudaStream_t stream);
  /**
   * Alltoall(v) of strided or index-selected rows of `row_bytes` bytes with the pack / unpack fused in
   * (sequence <-> head transposition, expert dispatch / combine).  Strides in bytes.
   */
  void exchange_rows(const std::vector<internal::device::RowArgs>& ranks, size_t row_bytes, size_t send_row_stride,
                     size_t recv_row_stride, cudaStream_t stream);
  /** Enqueue point-to-point transfers that progress together. */
  void p2p(const std::vector<internal::device::P2PDesc>& items, cudaStream_t stream);

  /** Collective allocation of symmetric memory (multicast-bound when possible). Returns this rank's pointer. */
  void* symm_alloc(size_t bytes);
  void symm_free(void* ptr);
  /**
   * Make a device buffer addressable by every rank of the communicator, so that reduce_scatter (as send
   * buffer) and allgather / alltoall / bcast (as receive buffer) run on it without staging.  Collective:
   * every rank calls it, in the same order, each with its own buffer (sizes may differ).  Memory from
   * cudaMalloc is shared through CUDA IPC handles; memory from symm_alloc() is already shared (and is
   * registered automatically when it is allocated).  Returns the window index, or -1 when some rank's
   * memory could not be shared (then no rank registers it and the buffer keeps using the staging path).
   * Role: ncclCommRegister behind Al::RegisterMemory (src/nccl_impl.cpp:83-109 of the reference).
   */
  int register_buffer(void* ptr, size_t bytes);
  /** Collective: forget a registered buffer (must be called before the memory is freed). */
  void unregister_buffer(void* ptr);
  /** Emulation: the buffers of all ranks at once (one process, one device). */
  int register_buffers_emulated(const std::vector<void*>& ptrs, size_t bytes);
  /** Window containing [ptr, ptr+bytes) of local rank `local_rank`, or -1; *offset = distance from its start. */
  int find_window(const void* ptr, size_t bytes, size_t* offset, int local_rank = 0) const;
  /**
   * Guard mode (tuning().debug_guard / AL_DEBUG_GUARD=1): every symm_alloc block carries a 4 KiB region of a
   * known pattern before and after the user's bytes.  Synchronises the device and throws al_exception if any
   * guard of this rank's blocks was overwritten (naming block, side and distance).  symm_free runs it too.
   */
  void check_guards() const;
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
  /**
   * Latency breakdown: with `on`, the small-message kernels of this communicator record %globaltimer at
   * entry / data sent / first data seen / exit into four device words; read_stamps() synchronises the
   * device and returns them (nanoseconds).  Off by default: the kernels then only test a null pointer.
   */
  void enable_stamps(bool on);
  void read_stamps(uint64_t out[4]) const;
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
