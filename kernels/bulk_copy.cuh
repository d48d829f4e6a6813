// Bulk asynchronous copies (the sm_90+/sm_100 copy engine reached with
// cp.async.bulk) driven by ONE thread per CTA through a ring of shared-memory
// tiles: global -> shared (completion on an mbarrier), shared -> global
// (completion through bulk groups).  The source is always this GPU's own
// memory; the destinations may be peer-mapped memory of other GPUs, which the
// engine reaches with ordinary one-destination stores over NVLink.
//
// Every wait in here is bounded.  A wait on an mbarrier that runs out returns
// false to the caller after the copies already in flight have drained, so the
// shared memory is quiet when the kernel returns.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "al/config.hpp"

namespace Al {
namespace internal {
namespace device {
namespace bulk {

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
/** Makes freshly initialised barriers visible to the copy engine. */
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
/** Orders earlier generic-proxy accesses (flag acquires, plain stores) before later copy-engine accesses and back. */
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
/** Bounded wait for the phase of `parity` to complete. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint64_t timeout_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  uint64_t t0;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (unsigned spins = 0;; ++spins) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((spins & 255) == 255) {
      uint64_t t;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
      if (t - t0 > timeout_ns) return false;
    }
  }
}

/** global (this GPU) -> shared, `bytes` a multiple of 16, both addresses 16-byte aligned. */
__device__ __forceinline__ void g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
/** shared -> global (local or peer-mapped), same alignment rules; completion tracked by the bulk group. */
__device__ __forceinline__ void s2g(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
/** At most N groups may still be READING their shared-memory source. */
template <int N>
__device__ __forceinline__ void wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
/** Every committed store has been performed. */
__device__ __forceinline__ void wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

/**
 * Ring of NBUF tiles of TILE bytes with one mbarrier each.  `parity` bit s is
 * the phase the next use of tile s has to wait for; it lives in a register of
 * the driving thread for the whole kernel.
 */
template <int NBUF, int TILE>
struct Ring {
  uint32_t tiles;    ///< shared address of tile 0 (1024-byte aligned)
  uint32_t bars;     ///< shared address of barrier 0
  uint32_t parity;

  __device__ __forceinline__ uint32_t tile(int s) const { return tiles + (uint32_t)s * TILE; }
  __device__ __forceinline__ uint32_t bar(int s) const { return bars + (uint32_t)s * 8; }

  /** Called by the driving thread once, before the first copy. */
  __device__ __forceinline__ void init(void* tile_mem, void* bar_mem) {
    tiles = smem_addr(tile_mem);
    bars = smem_addr(bar_mem);
    parity = 0;
    for (int s = 0; s < NBUF; ++s) mbar_init(bar(s), 1);
    fence_barrier_init();
  }
};

/**
 * One tile of a transfer list: `bytes` from local `src` to `ndst` destinations
 * (dst[0..ndst)).  A functor `F(t, Tile&)` describes tile number t.
 */
struct Tile {
  const char* src;
  char* dst[AL_MAX_DEVICE_RANKS];
  int ndst;
  uint32_t bytes;
};

/**
 * Stream `ntiles` tiles through the ring: loads run NBUF-1 tiles ahead of the
 * stores.  Called by the driving thread only.  On return every store has been
 * performed (bulk group wait) and ordered before later generic-proxy accesses
 * of this thread.  Returns false when a load did not complete in time.
 */
template <int NBUF, int TILE, typename F>
__device__ __forceinline__ bool stream_tiles(Ring<NBUF, TILE>& ring, size_t ntiles, F&& describe, uint64_t timeout_ns) {
  if (ntiles == 0) return true;
  fence_proxy_async();  // flag acquires / earlier plain accesses before the engine touches the data
  Tile tl;
  auto load = [&](size_t t) {
    describe(t, tl);
    const int s = (int)(t % NBUF);
    mbar_expect_tx(ring.bar(s), tl.bytes);
    g2s(ring.tile(s), tl.src, tl.bytes, ring.bar(s));
  };
  const size_t ahead = ntiles < (size_t)(NBUF - 1) ? ntiles : (size_t)(NBUF - 1);
  for (size_t t = 0; t < ahead; ++t) load(t);
  bool ok = true;
  for (size_t i = 0; i < ntiles; ++i) {
    const int s = (int)(i % NBUF);
    if (!mbar_wait(ring.bar(s), (ring.parity >> s) & 1u, timeout_ns)) { ok = false; break; }
    ring.parity ^= 1u << s;
    describe(i, tl);
    for (int d = 0; d < tl.ndst; ++d) s2g(tl.dst[d], ring.tile(s), tl.bytes);
    commit();
    const size_t j = i + NBUF - 1;  // goes into the tile that store group i-1 read from
    if (j < ntiles) {
      wait_read<1>();
      load(j);
    }
  }
  wait_all();
  fence_proxy_async();
  return ok;
}

}  // namespace bulk
}  // namespace device
}  // namespace internal
}  // namespace Al
