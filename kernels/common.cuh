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
__device__ __forceinline__ void arrive_and_post(const Workspace& ws, int rank, size_t off, int counter_idx,
                                                unsigned group, uint64_t epoch, bool with_meta, int meta_par,
                                                uint64_t meta_value) {
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    int last = 1;
    if (group > 1) {
      __threadfence();  // this CTA's writes before the arrival count
      unsigned* ctr = (unsigned*)flag_slot(ws.flags[rank], FlagLayout::off_arrive, counter_idx + 4 * (int)(epoch & 1));
      last = atomicInc(ctr, group - 1) == group - 1;
      if (last) __threadfence();  // other CTAs' writes before the flag stores
    }
    s_last = last;
  }
  __syncthreads();
  if (s_last && threadIdx.x < ws.p) {
    const int dst = threadIdx.x;
    if (with_meta)
      st_relaxed_sys(flag_slot(ws.flags[dst], FlagLayout::off_meta, meta_par * kMaxRanks + rank), meta_value);
    st_release_sys(flag_slot(ws.flags[dst], off, rank), epoch);
  }
}

/** Every CTA waits until all ranks posted `epoch` in this rank's array `off`.
 *  Returns false (block-uniform) after a time-out, which has been reported. */
__device__ __forceinline__ bool wait_all(const Workspace& ws, int rank, size_t off, uint32_t where,
                                         uint64_t epoch, uint64_t timeout_ns) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < ws.p) {
    uint64_t seen = 0;
    if (!wait_flag(flag_slot(ws.flags[rank], off, threadIdx.x), epoch, timeout_ns, &seen)) {
      report_timeout(ws, rank, threadIdx.x, where, epoch, seen);
      s_ok = 0;
    }
  }
  __syncthreads();
  return s_ok != 0;
}

}  // namespace device
}  // namespace internal
}  // namespace Al
