/**
 * @file rma.hpp
 * One-sided extension on device communicators: attach a peer's buffer, put
 * into it, and order accesses with notify / wait / sync.
 *
 * Parity: Al::ext of the reference (include/Al.hpp:1916-2001,
 * include/aluminum/mpi_cuda_impl.hpp:62-107, mpi_cuda/rma.hpp:66-183,
 * rma_ipc.hpp:152-328, rma_self.hpp, rma_null.hpp).  Differences:
 *   - Put is a grid of SM stores into the peer-mapped buffer (no copy engine);
 *   - Notify / Wait / Sync are a release store to / a bounded acquire wait on a
 *     counter in the peer's symmetric flag area, enqueued on the
 *     communicator's stream, with no host handshake and no progress-engine
 *     state (the reference's states never signal completion,
 *     rma_ipc.hpp:53-57 vs rma.hpp:149-168);
 *   - buffers from comm.symm_alloc() need no handle exchange; other device
 *     allocations are shared with cudaIpc handles.
 * Attach / Detach are collective per pair: both ranks must call them for each
 * other in matching order.  `peer < 0` is the null peer (every call is a
 * no-op), `peer == rank` the self connection.
 */
#pragma once
#include "al/device/communicator.hpp"

namespace Al {
namespace internal {
namespace rma {
void* attach(void* local_buf, int peer, DeviceCommunicator& comm);
void detach(void* remote_buf, int peer, DeviceCommunicator& comm);
void notify(int peer, DeviceCommunicator& comm);
void wait(int peer, DeviceCommunicator& comm);
void put(const void* src, int dest, void* dest_remote, size_t bytes, DeviceCommunicator& comm);
void get(void* dst, int src_rank, const void* src_remote, size_t bytes, DeviceCommunicator& comm);
/** Drop the bookkeeping (signal counters, imported mappings) kept for a communicator that is going away. */
void forget(const void* comm_impl) noexcept;
}  // namespace rma
}  // namespace internal

namespace ext {

/** Exchange buffer addresses with `peer`; returns the address of the peer's buffer in this process (nullptr if the peer passed nullptr). */
template <typename T>
T* AttachRemoteBuffer(T* local_buf, int peer, DeviceCommunicator& comm) {
  return static_cast<T*>(internal::rma::attach(local_buf, peer, comm));
}
template <typename T>
void DetachRemoteBuffer(T* remote_buf, int peer, DeviceCommunicator& comm) {
  internal::rma::detach(remote_buf, peer, comm);
}
/** Signal `peer` once everything enqueued so far on the communicator's stream has completed. */
inline void Notify(int peer, DeviceCommunicator& comm) { internal::rma::notify(peer, comm); }
/** Make the communicator's stream wait for the matching Notify from `peer`. */
inline void Wait(int peer, DeviceCommunicator& comm) { internal::rma::wait(peer, comm); }
/** Notify + Wait: both sides have reached this point of their streams. */
inline void Sync(int peer, DeviceCommunicator& comm) {
  internal::rma::notify(peer, comm);
  internal::rma::wait(peer, comm);
}
inline void Sync(const int* peers, int num_peers, DeviceCommunicator& comm) {
  for (int i = 0; i < num_peers; ++i) internal::rma::notify(peers[i], comm);
  for (int i = 0; i < num_peers; ++i) internal::rma::wait(peers[i], comm);
}
/** Copy `count` elements from local `srcbuf` into `destbuf`, an address obtained from AttachRemoteBuffer for `dest`. */
template <typename T>
void Put(const T* srcbuf, int dest, T* destbuf, size_t count, DeviceCommunicator& comm) {
  internal::rma::put(srcbuf, dest, destbuf, count * sizeof(T), comm);
}

/**
 * The other direction: copy `count` elements out of `srcbuf`, an address obtained from
 * AttachRemoteBuffer for rank `src`, into local `destbuf`.  Stream-ordered like Put; the owner of
 * `srcbuf` tells the reader when the data may be read (Notify / Wait or Sync) and learns the same
 * way when the read is over.  The reference's interface stops at Put; its north star (put / get over
 * CUDA IPC) and DistConv-style pull patterns want this verb.  Loads over NVLink stall the issuing
 * threads (stores are posted), so a Get moves about half of a Put's bandwidth: prefer Put where the
 * producer can drive the transfer.
 */
template <typename T>
void Get(T* destbuf, int src, const T* srcbuf, size_t count, DeviceCommunicator& comm) {
  internal::rma::get(destbuf, src, srcbuf, count * sizeof(T), comm);
}

}  // namespace ext
}  // namespace Al
