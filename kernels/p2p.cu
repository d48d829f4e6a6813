// Point-to-point transfers over peer-mapped mailboxes: Send, Recv, SendRecv and
// MultiSendRecv are one kernel walking a list of transfer descriptors.
//
// Every ordered pair (src -> dst) owns a two-slot ring in dst's mailbox area.
// The sender waits for a free slot (its local `acked` word, advanced remotely
// by the receiver), stores the piece straight into the receiver's slot over
// NVLink and then advances the receiver's `sent` word with a release store;
// the receiver polls its local `sent` word, copies the piece to the user
// buffer and advances the sender's `acked` word.  Both sides therefore only
// ever poll their own memory.  Messages larger than a slot are pipelined
// piece by piece through the two slots.  Role of ncclSend / ncclRecv groups in
// the reference (include/aluminum/nccl_impl.hpp:957-1077).
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

/** Block-uniform bounded wait on one local word; thread 0 polls. */
__device__ __forceinline__ bool cta_wait_word(const uint64_t* word, uint64_t target, uint64_t timeout_ns,
                                              const Workspace& ws, int rank, int peer, uint32_t where) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) {
    uint64_t seen = 0;
    s_ok = wait_flag(word, target, timeout_ns, &seen) ? 1 : 0;
    if (!s_ok) report_timeout(ws, rank, peer, where, target, seen);
  }
  __syncthreads();
  const int ok = s_ok;
  __syncthreads();
  return ok != 0;
}

/** All CTAs of an item's group call this after their share of a piece; the last one runs `post`. */
template <typename Post>
__device__ __forceinline__ void group_arrive(uint64_t* counter_slot, unsigned group, Post post) {
  __syncthreads();
  if (threadIdx.x == 0) {
    bool last = true;
    __threadfence_system();  // remote stores of this CTA before the arrival count
    if (group > 1) last = atomicInc((unsigned*)counter_slot, group - 1) == group - 1;
    if (last) {
      __threadfence_system();
      post();
    }
  }
}

__global__ void __launch_bounds__(512) p2p_kernel(const __grid_constant__ P2PParams P) {
  const Workspace& ws = P.ws;
  const unsigned group = (unsigned)P.ctas_per_item;
  const int item = (int)(blockIdx.x / group);
  const unsigned part = blockIdx.x % group;
  if (item >= P.nitems) return;
  const int me = P.owner[item], peer = P.peer[item];
  if (poisoned(ws, me)) return;
  const size_t slot = ws.mbox_slot_bytes;
  const size_t bytes = P.bytes[item];
  const size_t pieces = bytes == 0 ? 1 : (bytes + slot - 1) / slot;
  uint64_t* myflags = ws.flags[me];
  // Arrivals are counted per piece parity: the credit gate of piece n depends on the post of
  // piece n-2, so a CTA is never more than one unposted piece ahead of its slowest sibling.
  uint64_t* arrive2[2] = {flag_slot(myflags, FlagLayout::off_p2p_arrive, item),
                          flag_slot(myflags, FlagLayout::off_p2p_arrive, item + P2PParams::kMaxItems)};

  if (P.is_send[item]) {
    const uint64_t base = P.base[item];  // pieces already sent to this peer by earlier launches
    const uint64_t* acked = flag_slot(myflags, FlagLayout::off_p2p_acked, peer);
    uint64_t* sent_remote = flag_slot(ws.flags[peer], FlagLayout::off_p2p_sent, me);
    const char* src = (const char*)P.sbuf[item];
    for (size_t k = 0; k < pieces; ++k) {
      const uint64_t n = base + k;
      // a slot is free once the receiver consumed piece n-2
      if (n >= 2 && !cta_wait_word(acked, n - 1, P.timeout_ns, ws, me, peer, 3)) return;
      const size_t off = k * slot, len = bytes > off ? (bytes - off < slot ? bytes - off : slot) : 0;
      size_t lo, hi;
      split_range(len, part, group, 16, lo, hi);
      char* dst = ws.mbox[peer] + ((size_t)me * 2 + (n & 1)) * slot;
      if (hi > lo) cta_copy(dst + lo, src + off + lo, hi - lo, false);
      group_arrive(arrive2[n & 1], group, [&] {
        st_release_sys(sent_remote, n + 1);
      });
    }
  } else {
    const uint64_t base = P.base[item];  // pieces already received from this peer
    const uint64_t* sent = flag_slot(myflags, FlagLayout::off_p2p_sent, peer);
    uint64_t* acked_remote = flag_slot(ws.flags[peer], FlagLayout::off_p2p_acked, me);
    char* dstbuf = (char*)P.rbuf[item];
    for (size_t k = 0; k < pieces; ++k) {
      const uint64_t n = base + k;
      if (!cta_wait_word(sent, n + 1, P.timeout_ns, ws, me, peer, 4)) return;
      const size_t off = k * slot, len = bytes > off ? (bytes - off < slot ? bytes - off : slot) : 0;
      size_t lo, hi;
      split_range(len, part, group, 16, lo, hi);
      const char* src = ws.mbox[me] + ((size_t)peer * 2 + (n & 1)) * slot;
      if (hi > lo) cta_copy(dstbuf + off + lo, src + lo, hi - lo, true);
      group_arrive(arrive2[n & 1], group, [&] {
        st_release_sys(acked_remote, n + 1);
      });
    }
  }
}

}  // namespace

void launch_p2p(const P2PParams& P, int threads, int cooperative, cudaStream_t stream) {
  if (P.nitems <= 0) return;
  dim3 grid((unsigned)(P.nitems * P.ctas_per_item));
  void* args[] = {(void*)&P};
  if (cooperative)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)p2p_kernel, grid, dim3((unsigned)threads), args, 0, stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)p2p_kernel, grid, dim3((unsigned)threads), args, 0, stream));
}

}  // namespace device
}  // namespace internal
}  // namespace Al
