// Device-side building blocks shared by every collective kernel: system-scope
// flag accesses, bounded waits with status reporting, the "last CTA posts"
// arrival pattern, CTA-wide copies and element-wise reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "al/base.hpp"
#include "al/device/params.hpp"

namespace Al {
namespace internal {
namespace device {

// ---------------------------------------------------------------------------
// system-scope memory operations
// ---------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint64_t* p, uint64_t v) {
  asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ uint64_t ld_acquire_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t ld_relaxed_sys(const uint64_t* p) {
  uint64_t v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

/** Latency breakdown: one thread of the launch records the global timer at point `i` (0..3) when asked to. */
__device__ __forceinline__ void stamp(const Workspace& ws, int i) {
  if (ws.stamps && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) ws.stamps[i] = global_ns();
}

__device__ __forceinline__ uint64_t make_epoch(uint64_t seq, uint64_t sub) { return (seq << 24) | sub; }

__device__ __forceinline__ uint64_t* flag_slot(uint64_t* area, size_t off, int idx) {
  return area + off + (size_t)idx * FlagLayout::stride;
}

// ---------------------------------------------------------------------------
// failure reporting
// ---------------------------------------------------------------------------
/** Record the first failure of this communicator: device-local word (so that
 *  later kernels return at once) and the pinned host record. */
__device__ __forceinline__ void report_timeout(const Workspace& ws, int rank, int peer, uint32_t where,
                                               uint64_t epoch, uint64_t seen) {
  unsigned long long* local = (unsigned long long*)flag_slot(ws.flags[rank], FlagLayout::off_status, 0);
  if (atomicCAS(local, 0ull, (unsigned long long)kStatusTimeout) == 0ull) {
    DeviceStatus* s = ws.status;
    if (s) {
      s->rank = (uint32_t)rank;
      s->peer = (uint32_t)peer;
      s->where = where;
      s->epoch = epoch;
      s->seen = seen;
      __threadfence_system();
      s->code = kStatusTimeout;
      __threadfence_system();
    }
  }
}

/** Record a failure other than a time-out (same rules: first one wins, later kernels return at once). */
__device__ __forceinline__ void report_status(const Workspace& ws, int rank, uint32_t code, int peer, uint32_t where,
                                              uint64_t epoch, uint64_t seen) {
  unsigned long long* local = (unsigned long long*)flag_slot(ws.flags[rank], FlagLayout::off_status, 0);
  if (atomicCAS(local, 0ull, (unsigned long long)code) == 0ull) {
    DeviceStatus* s = ws.status;
    if (s) {
      s->rank = (uint32_t)rank;
      s->peer = (uint32_t)peer;
      s->where = where;
      s->epoch = epoch;
      s->seen = seen;
      __threadfence_system();
      s->code = code;
      __threadfence_system();
    }
  }
}

__device__ __forceinline__ bool poisoned(const Workspace& ws, int rank) {
  return ld_relaxed_sys(flag_slot(ws.flags[rank], FlagLayout::off_status, 0)) != 0;
}

/**
 * Spin until *slot >= epoch.  Gives up after timeout_ns (checked with the
 * global nanosecond timer after an initial burst of cheap polls).
 */
__device__ __forceinline__ bool wait_flag(const uint64_t* slot, uint64_t epoch, uint64_t timeout_ns,
                                          uint64_t* seen_out) {
  uint64_t v = ld_acquire_sys(slot);
  if (v >= epoch) return true;
  unsigned spins = 0;
  uint64_t t0 = 0;
  for (;;) {
    v = ld_acquire_sys(slot);
    if (v >= epoch) return true;
    ++spins;
    if (spins > 32) {
      __nanosleep(spins > 4096 ? 400 : 40);
      if (t0 == 0) t0 = global_ns();
      else if ((spins & 63) == 0 && global_ns() - t0 > timeout_ns) {
        *seen_out = v;
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// handshakes
// ---------------------------------------------------------------------------
/**
 * Called by every thread of every CTA of a group of `group` CTAs of `rank` once
 * the CTA's share of the preceding writes is issued.  The last CTA to arrive stores `epoch` into
 * slot [rank] of every rank's flag array `off` (optionally after publishing
 * `meta_value` into the meta word of parity `meta_par`).
 *
 * Consecutive rounds of one kernel carry consecutive epochs and count their arrivals in
 * two counters chosen by the epoch's low bit.  In every schedule of this library a CTA can
 * only be two rounds ahead of the slowest CTA of its group once the round in between has been
 * posted (the gate of round k+2 depends, through the peers, on the post of round k), so the
 * arrivals of at most two neighbouring rounds are ever in flight and a fast CTA's arrival
 * for round k+1 can never complete the count of round k.
 */
__device__ __forceinline__ void arrive_and_post_ctr(const Workspace& ws, int rank, size_t off, unsigned* ctr,
                                                    unsigned group, uint64_t epoch, bool with_meta, int meta_par,
                                                    uint64_t meta_value, uint64_t meta_proto = 0, int word = 0) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    int last = 1;
    if (group > 1) {
      __threadfence();  // this CTA's writes before the arrival count
      last = atomicInc(ctr, group - 1) == group - 1;
      if (last) __threadfence();  // other CTAs' writes before the flag stores
    }
    s_last = last;
  }
  __syncthreads();
  if (s_last && threadIdx.x < ws.p) {
    const int dst = threadIdx.x;
    if (with_meta) {
      uint64_t* m = flag_slot(ws.flags[dst], FlagLayout::off_meta, meta_par * kMaxRanks + rank);
      st_relaxed_sys(m + kMetaChunks, meta_value);
      if (meta_proto) st_relaxed_sys(m + kMetaProto, meta_proto);
    }
    st_release_sys(flag_slot(ws.flags[dst], off, rank) + word, epoch);
  }
}

__device__ __forceinline__ void arrive_and_post(const Workspace& ws, int rank, size_t off, int counter_idx,
                                                unsigned group, uint64_t epoch, bool with_meta, int meta_par,
                                                uint64_t meta_value, uint64_t meta_proto = 0) {
  unsigned* ctr = (unsigned*)flag_slot(ws.flags[rank], FlagLayout::off_arrive, counter_idx + 4 * (int)(epoch & 1));
  arrive_and_post_ctr(ws, rank, off, ctr, group, epoch, with_meta, meta_par, meta_value, meta_proto);
}

/**
 * The same for kernels that keep up to `depth` (<= kRingDepth) rounds in flight: one counter per CTA group
 * (0..2) and ring slot.  Valid while no CTA can be `depth` rounds ahead of the slowest CTA of its group,
 * which the ring-pipelined kernels guarantee by gating round c on the completion of round c - depth.
 */
__device__ __forceinline__ void arrive_and_post_ring(const Workspace& ws, int rank, size_t off, int group_id, uint64_t round,
                                                     int depth, unsigned group, uint64_t epoch, bool with_meta, int meta_par,
                                                     uint64_t meta_value, uint64_t meta_proto = 0, int word = 0) {
  unsigned* ctr = (unsigned*)(ws.flags[rank] + FlagLayout::off_ring_arrive + (size_t)group_id * kRingDepth + (size_t)(round % (uint64_t)depth));
  arrive_and_post_ctr(ws, rank, off, ctr, group, epoch, with_meta, meta_par, meta_value, meta_proto, word);
}

/** Every CTA waits until all ranks posted `epoch` in this rank's array `off`.
 *  Returns false (block-uniform) after a time-out, which has been reported. */
__device__ __forceinline__ bool wait_all(const Workspace& ws, int rank, size_t off, uint32_t where,
                                         uint64_t epoch, uint64_t timeout_ns, int word = 0) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < ws.p) {
    uint64_t seen = 0;
    if (!wait_flag(flag_slot(ws.flags[rank], off, threadIdx.x) + word, epoch, timeout_ns, &seen)) {
      report_timeout(ws, rank, threadIdx.x, where, epoch, seen);
      s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}

// ---------------------------------------------------------------------------
// protocol agreement
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint64_t proto_word(ProtoTag tag, int kind, int variant = 0) {
  return ((uint64_t)tag << 8) | (uint64_t)(kind & 0xff) | ((uint64_t)(variant & 0xff) << 16);
}

/**
 * "I have entered operation `seq`": one CTA (the caller picks it) stores this rank's protocol word
 * and buffer descriptors into every rank's meta slot and then the B flag.  The stream order of the
 * poster guarantees that its earlier work on its buffers is complete, so peers that see the flag may
 * write into (or read from) its registered buffers.  Nobody has to wait for it: kernels that go
 * through staging post it and carry on.
 */
__device__ __forceinline__ void post_entered(const Workspace& ws, int rank, uint64_t seq, uint64_t proto,
                                             uint64_t recv_desc, uint64_t send_desc) {
  if (threadIdx.x < ws.p) {
    const int dst = threadIdx.x;
    uint64_t* m = flag_slot(ws.flags[dst], FlagLayout::off_meta, (int)(seq & 1) * kMaxRanks + rank);
    st_relaxed_sys(m + kMetaProto, proto);
    st_relaxed_sys(m + kMetaRecvDesc, recv_desc);
    st_relaxed_sys(m + kMetaSendDesc, send_desc);
    st_release_sys(flag_slot(ws.flags[dst], FlagLayout::off_B, rank), make_epoch(seq, 1));
  }
}

/**
 * After a wait that made every rank's protocol word visible: do all ranks run the protocol `mine`?
 * Block-uniform answer.  On disagreement the failure is recorded as kStatusMismatch (peer = first
 * rank that differs, seen = its word) and this rank's A and C flags are pushed to the operation's
 * last possible epoch, so that a peer which is waiting for them under the other protocol wakes up,
 * compares the words as well and returns - nobody is left to a time-out.
 */
__device__ __forceinline__ bool protocols_agree(const Workspace& ws, int rank, uint64_t seq, uint64_t mine) {
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = -1;
  __syncthreads();
  if (threadIdx.x < ws.p) {
    const uint64_t* m = flag_slot(ws.flags[rank], FlagLayout::off_meta, (int)(seq & 1) * kMaxRanks + threadIdx.x);
    if (ld_relaxed_sys(m + kMetaProto) != mine) atomicMax(&s_bad, (int)threadIdx.x);
  }
  __syncthreads();
  const int bad = s_bad;
  if (bad < 0) return true;
  if (threadIdx.x < ws.p) {
    if (threadIdx.x == 0) {
      const uint64_t* m = flag_slot(ws.flags[rank], FlagLayout::off_meta, (int)(seq & 1) * kMaxRanks + bad);
      report_status(ws, rank, kStatusMismatch, bad, 7, mine, ld_relaxed_sys(m + kMetaProto));
    }
    const uint64_t last = make_epoch(seq, 0xFFFFFE);
    st_release_sys(flag_slot(ws.flags[threadIdx.x], FlagLayout::off_A, rank), last);
    st_release_sys(flag_slot(ws.flags[threadIdx.x], FlagLayout::off_B, rank), last);
    st_release_sys(flag_slot(ws.flags[threadIdx.x], FlagLayout::off_B, rank) + 1, last);  // odd chunks of the pipelined NVLS allreduce
    st_release_sys(flag_slot(ws.flags[threadIdx.x], FlagLayout::off_C, rank), last);
  }
  __syncthreads();
  return false;
}

}  // namespace device
}  // namespace internal
}  // namespace Al
