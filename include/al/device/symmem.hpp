/**
 * @file symmem.hpp
 * Symmetric device memory: an allocation made collectively by the ranks of a
 * group such that every rank can address every other rank's copy, optionally
 * with an NVLink-multicast (NVLS) alias that addresses all copies at once.
 *
 * This is the memory plane that replaces what NCCL sets up inside
 * ncclCommInitRank / ncclCommRegister for the reference
 * (src/nccl_impl.cpp:46-60,83-109) and the cudaIpc* attach of its RMA
 * extension (include/aluminum/mpi_cuda/rma_ipc.hpp:194-229).
 *
 * Backings:
 *   vmm       cuMemCreate with a POSIX-fd shareable handle, descriptors passed
 *             over the control plane (SCM_RIGHTS), cuMemMap on every rank;
 *             cuMulticastCreate/AddDevice/BindMem for the multicast alias.
 *   ipc       cudaMalloc + cudaIpcGetMemHandle/OpenMemHandle (no multicast);
 *             chosen with AL_DEV_SYMM=ipc or when the vmm path is unavailable.
 *   emulated  all ranks live in this process on one device: plain cudaMalloc
 *             per rank (used to test the kernels on a single GPU).
 */
#pragma once
#include <memory>
#include <vector>

#include "al/bootstrap.hpp"
#include "al/cuda/cuda.hpp"
#include "al/device/params.hpp"

namespace Al {
namespace internal {
namespace device {

class SymmBlock {
 public:
  ~SymmBlock();
  SymmBlock(const SymmBlock&) = delete;
  SymmBlock& operator=(const SymmBlock&) = delete;

  /** Collective over `group`: every rank contributes `bytes` (same value everywhere). */
  static std::unique_ptr<SymmBlock> create(const Group& group, size_t bytes, bool want_multicast);
  /** All `p` ranks in this process on the current device. */
  static std::unique_ptr<SymmBlock> create_emulated(int p, size_t bytes);

  size_t bytes() const { return bytes_; }
  int size() const { return p_; }
  /** Address of rank r's copy in this process. */
  void* peer(int r) const { return peer_[r]; }
  /** Multicast alias (nullptr when unavailable). */
  void* mc() const { return mc_; }
  const char* backing() const { return backing_; }

 private:
  SymmBlock() = default;
  bool try_vmm(const Group& group, size_t bytes, bool want_multicast);
  void make_ipc(const Group& group, size_t bytes);

  size_t bytes_ = 0, mapped_bytes_ = 0;
  int p_ = 0, me_ = 0;
  void* peer_[kMaxRanks] = {};
  void* mc_ = nullptr;
  const char* backing_ = "none";
  // vmm
  std::vector<CUmemGenericAllocationHandle> handles_;
  CUmemGenericAllocationHandle mc_handle_ = 0;
  bool mc_bound_ = false;
  int device_ = 0;
  // ipc / emulated
  std::vector<void*> owned_;       // cudaMalloc'ed by this process
  std::vector<void*> ipc_opened_;  // opened peer handles
};

/** Process-level facts about the GPUs, for al_info and algorithm selection. */
struct Topology {
  int device_count = 0;
  int device = -1;
  std::string name;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t total_mem = 0;
  bool multicast_supported = false;
  bool vmm_fd_supported = false;
  std::vector<int> p2p_access;         ///< [device_count] can the current device access device i
  std::vector<int> p2p_native_atomics; ///< [device_count]
  std::string describe() const;
};
Topology discover_topology();

}  // namespace device
}  // namespace internal
}  // namespace Al
