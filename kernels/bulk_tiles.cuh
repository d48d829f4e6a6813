// Where every tile of the bulk-copy kernels comes from and goes to.
//
// Plain index arithmetic, usable from device code and from host code: the unit
// tests execute these plans on host memory for many (ranks, sizes, grids) and
// check that every byte arrives exactly where the collective's definition puts
// it, which is the part of the kernels that can be verified without a GPU.
// All quantities are BYTES; slices, slots and chunk sizes are multiples of 16.
#pragma once
#include <cstddef>
#include <cstdint>

#if defined(__CUDACC__)
#define AL_HD __host__ __device__ __forceinline__
#else
#define AL_HD inline
#endif

namespace Al {
namespace internal {
namespace device {
namespace plan {

/** Sub-range [lo, hi) of [0, len) owned by part i of n; boundaries are multiples of 16 (len itself is one). */
AL_HD void split16(size_t len, unsigned i, unsigned n, size_t& lo, size_t& hi) {
  size_t per = (len + n - 1) / n;
  per = (per + 15) / 16 * 16;
  lo = per * i;
  if (lo > len) lo = len;
  hi = lo + per;
  if (hi > len) hi = len;
}

AL_HD size_t clamp(size_t count, size_t lo, size_t cap) {
  if (count <= lo) return 0;
  const size_t r = count - lo;
  return r < cap ? r : cap;
}

/** One transfer: `bytes` from offset `src` of the source buffer to offset `dst` of the buffer of rank `peer`. */
struct Move {
  size_t src;
  size_t dst;
  uint32_t bytes;
  int peer;  ///< destination rank; -1: every rank (allgather publish), rotated from rank+1
};

/**
 * The work of one CTA (`part` of `nparts`) in one chunk of a staged, pipelined
 * operation: `seg` bytes starting at `lo` of the chunk's range, cut into tiles.
 */
struct Share {
  size_t base;   ///< first byte of the chunk inside a rank slice
  size_t lo;     ///< first byte of this CTA's share inside the chunk
  size_t seg;    ///< bytes of this CTA's share
  size_t tiles;  ///< tiles per source / destination
};

AL_HD Share share_of(size_t slice, size_t slot, uint64_t chunk, unsigned part, unsigned nparts, size_t tile) {
  Share s;
  s.base = chunk * slot;
  const size_t len = clamp(slice, s.base, slot);
  size_t hi;
  split16(len, part, nparts, s.lo, hi);
  s.seg = hi - s.lo;
  s.tiles = (s.seg + tile - 1) / tile;
  return s;
}

AL_HD uint32_t tile_bytes(const Share& s, size_t k, size_t tile) {
  const size_t off = k * tile;
  return (uint32_t)(s.seg - off < tile ? s.seg - off : tile);
}

// ---- staged pipeline (bulk_pipeline.cu) -------------------------------------------------
// Staging half of a rank: p slots of `cap` bytes, slot [r] holds what rank r published.

/** Allgather publish, tile k: source = the rank's send buffer, destination = slot [rank] of every rank. */
AL_HD Move ag_publish(const Share& s, size_t k, int rank, size_t cap, size_t tile) {
  Move m;
  m.src = s.base + s.lo + k * tile;
  m.dst = (size_t)rank * cap + s.lo + k * tile;
  m.bytes = tile_bytes(s, k, tile);
  m.peer = -1;
  return m;
}

/** Number of tiles of a reduce_scatter / alltoall publish or an allgather / alltoall consume. */
AL_HD size_t fan_tiles(const Share& s, int p) { return s.tiles * (size_t)p; }

/** Reduce_scatter / alltoall publish, tile t: slice d of the send buffer goes to slot [rank] of rank d. */
AL_HD Move scatter_publish(const Share& s, size_t t, int rank, int p, size_t slice, size_t cap, size_t tile) {
  const int d = (rank + 1 + (int)(t % (size_t)p)) % p;
  const size_t k = t / (size_t)p;
  Move m;
  m.src = (size_t)d * slice + s.base + s.lo + k * tile;
  m.dst = (size_t)rank * cap + s.lo + k * tile;
  m.bytes = tile_bytes(s, k, tile);
  m.peer = d;
  return m;
}

/** Allgather / alltoall consume, tile t: slot [r] of the own staging half goes to slice r of the receive buffer. */
AL_HD Move gather_consume(const Share& s, size_t t, int p, size_t slice, size_t cap, size_t tile) {
  const int r = (int)(t % (size_t)p);
  const size_t k = t / (size_t)p;
  Move m;
  m.src = (size_t)r * cap + s.lo + k * tile;
  m.dst = (size_t)r * slice + s.base + s.lo + k * tile;
  m.bytes = tile_bytes(s, k, tile);
  m.peer = r;  // the rank whose data this is (the copy itself is local)
  return m;
}

}  // namespace plan
}  // namespace device
}  // namespace internal
}  // namespace Al
