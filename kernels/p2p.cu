// Point-to-point transfers: Send, Recv, SendRecv and MultiSendRecv are one kernel walking a list of
// transfer descriptors.  Role of ncclSend / ncclRecv groups in the reference
// (include/aluminum/nccl_impl.hpp:957-1077).
//
// Eager path (any buffer).  Every ordered pair (src -> dst) owns a ring of mailbox slots in dst's
// workspace.  The sender waits for a free slot (its local `acked` word, advanced remotely by the
// receiver), stores the piece straight into the receiver's slot over NVLink and then advances the
// receiver's `sent` word with a release store; the receiver polls its local `sent` word, copies the piece
// to the user buffer and advances the sender's `acked` word.  Both sides only ever poll their own memory.
// Messages larger than a slot are pipelined piece by piece through the ring.
//
// Rendezvous path (large messages).  From `rendezvous_bytes` on, the receiver first tells the sender
// where the data should go: it writes the descriptor of its buffer (window, offset; 0 = not registered)
// and the message's first piece number into the sender's `ready` slot.  If the buffer is registered the
// sender stores the whole message straight into it with all of its CTAs - no mailbox, no pieces, no
// copy-out - and posts `sent` once; the receiver only waits.  If not, both sides fall back to the ring.
// Both sides know the message size, so they agree on which protocol applies.
//
// Packet path (small messages, up to `ll_bytes`).  The data travels as 16-byte vectors {word, n+1, word, n+1}
// (n = the pair's piece number) into a ring of packet slots of its own; the receiver polls the vectors
// themselves, so there is no fence and no `sent` store behind the data - one NVLink trip instead of three.
// The receiver returns the slot's credit through `acked` as on the eager path; `sent` is not advanced, which
// is fine because every wait on it is a wait for "at least".
//
// CTA groups: every item is served by `ctas_per_item` CTAs; the one that finishes a piece last posts it.
// Arrivals are counted in two counters chosen by the piece's parity, and a CTA arrives for piece k only
// after piece k-2 has been posted (a local word the posting CTA writes), so a fast CTA can never complete
// the count of an earlier piece.  Every wait is bounded.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"
#include "packets.cuh"

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
  const uint64_t S = (uint64_t)ws.mbox_slots;
  const size_t bytes = P.bytes[item];
  const size_t pieces = bytes == 0 ? 1 : (bytes + slot - 1) / slot;
  const uint64_t base = P.base[item];  // pieces already moved between this pair in this direction
  uint64_t* myflags = ws.flags[me];
  uint64_t* arrive2[2] = {flag_slot(myflags, FlagLayout::off_p2p_arrive, item),
                          flag_slot(myflags, FlagLayout::off_p2p_arrive, item + P2PParams::kMaxItems)};
  uint64_t* posted = myflags + FlagLayout::off_p2p_posted + item;  // local: (launch << 32) | pieces of this item posted
  const uint64_t tag = P.launch << 32;
  // Arrive for piece k of this item only once piece k-2 has been posted (see the header).
  auto gate = [&](size_t k) {
    return k < 2 || cta_wait_word(posted, tag | (uint64_t)(k - 1), P.timeout_ns, ws, me, me, 3);
  };
  const bool rendezvous = bytes >= P.rendezvous_bytes && bytes > 0;
  const bool packets = bytes > 0 && bytes <= P.ll_bytes;
  uint32_t pflag = (uint32_t)(base + 1);  // epoch inside the packets; 0 is what fresh memory holds
  if (pflag == 0) pflag = 1;
  const size_t pgroups = (bytes + 15) / 16;
  const size_t ptid = (size_t)part * blockDim.x + threadIdx.x, pthreads = (size_t)group * blockDim.x;

  if (P.is_send[item]) {
    const uint64_t* acked = flag_slot(myflags, FlagLayout::off_p2p_acked, peer);
    uint64_t* sent_remote = flag_slot(ws.flags[peer], FlagLayout::off_p2p_sent, me);
    const char* src = (const char*)P.sbuf[item];
    if (packets) {
      if (base >= S && !cta_wait_word(acked, base - S + 1, P.timeout_ns, ws, me, peer, 3)) return;
      char* dst = ws.ll[peer] + kLLAreaBytes + ((size_t)me * S + (base % S)) * ws.p2p_ll_slot_bytes;
      for (size_t g = ptid; g < pgroups; g += pthreads)
        send_group(dst, g, load_group((const uint8_t*)src, g * 16, bytes), pflag);
      return;
    }
    if (rendezvous) {
      const uint64_t* ready = flag_slot(myflags, FlagLayout::off_p2p_ready, peer);
      if (!cta_wait_word(ready, base + 1, P.timeout_ns, ws, me, peer, 3)) return;
      const uint64_t desc = ld_relaxed_sys(ready + 1);
      if (desc != 0) {
        // straight into the receiver's registered buffer: one shot with every CTA of the group
        char* dst = P.windows->peer[(int)(desc >> 48) - 1][peer] + (size_t)(desc & ((uint64_t{1} << 48) - 1));
        size_t lo, hi;
        split_range(bytes, part, group, 16, lo, hi);
        if (hi > lo) cta_copy(dst + lo, src + lo, hi - lo, false);
        group_arrive(arrive2[base & 1], group, [&] { st_release_sys(sent_remote, base + pieces); });
        return;
      }
    }
    for (size_t k = 0; k < pieces; ++k) {
      const uint64_t n = base + k;
      // a slot is free once the receiver consumed piece n-S
      if (n >= S && !cta_wait_word(acked, n - S + 1, P.timeout_ns, ws, me, peer, 3)) return;
      const size_t off = k * slot, len = bytes > off ? (bytes - off < slot ? bytes - off : slot) : 0;
      size_t lo, hi;
      split_range(len, part, group, 16, lo, hi);
      char* dst = ws.mbox[peer] + ((size_t)me * S + (n % S)) * slot;
      if (hi > lo) cta_copy(dst + lo, src + off + lo, hi - lo, false);
      if (!gate(k)) return;
      group_arrive(arrive2[n & 1], group, [&] {
        st_release_sys(sent_remote, n + 1);
        *(volatile uint64_t*)posted = tag | (uint64_t)(k + 1);
      });
    }
  } else {
    const uint64_t* sent = flag_slot(myflags, FlagLayout::off_p2p_sent, peer);
    uint64_t* acked_remote = flag_slot(ws.flags[peer], FlagLayout::off_p2p_acked, me);
    char* dstbuf = (char*)P.rbuf[item];
    if (packets) {
      const char* slot_in = ws.ll[me] + kLLAreaBytes + ((size_t)peer * S + (base % S)) * ws.p2p_ll_slot_bytes;
      int bad = 0;
      for (size_t g = ptid; g < pgroups && !bad; g += pthreads) {
        uint4 v;
        if (recv_group(slot_in, g, pflag, v, ws, me, peer, base + 1, P.timeout_ns, 4)) store_group((uint8_t*)dstbuf, g * 16, bytes, v);
        else bad = 1;
      }
      if (__syncthreads_or(bad)) return;  // timed out (recorded): no credit is returned
      if (threadIdx.x == 0) {
        // every thread of this CTA has consumed its packets; the last CTA of the group frees the slot
        const bool last = group == 1 || atomicInc((unsigned*)arrive2[base & 1], group - 1) == group - 1;
        if (last) st_relaxed_sys(acked_remote, base + 1);
      }
      return;
    }
    if (rendezvous) {
      // tell the sender where the data goes (0: through the mailbox ring)
      if (part == 0 && threadIdx.x == 0) {
        uint64_t* ready_remote = flag_slot(ws.flags[peer], FlagLayout::off_p2p_ready, me);
        st_relaxed_sys(ready_remote + 1, P.rdesc[item]);
        st_release_sys(ready_remote, base + 1);
      }
      if (P.rdesc[item] != 0) {
        if (part == 0) {  // the data lands in place: wait for all of it, then return the credit of its pieces
          if (!cta_wait_word(sent, base + pieces, P.timeout_ns, ws, me, peer, 4)) return;
          if (threadIdx.x == 0) st_release_sys(acked_remote, base + pieces);
        }
        return;
      }
    }
    for (size_t k = 0; k < pieces; ++k) {
      const uint64_t n = base + k;
      if (!cta_wait_word(sent, n + 1, P.timeout_ns, ws, me, peer, 4)) return;
      const size_t off = k * slot, len = bytes > off ? (bytes - off < slot ? bytes - off : slot) : 0;
      size_t lo, hi;
      split_range(len, part, group, 16, lo, hi);
      const char* src = ws.mbox[me] + ((size_t)peer * S + (n % S)) * slot;
      if (hi > lo) cta_copy(dstbuf + off + lo, src + lo, hi - lo, true);
      if (!gate(k)) return;
      group_arrive(arrive2[n & 1], group, [&] {
        st_release_sys(acked_remote, n + 1);
        *(volatile uint64_t*)posted = tag | (uint64_t)(k + 1);
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
