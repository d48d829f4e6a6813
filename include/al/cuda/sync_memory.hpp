/**
 * @file sync_memory.hpp
 * Pool of pinned, device-visible 32-bit flag words, one per 128-byte line.
 * Parity: include/aluminum/cuda/sync_memory.hpp:46-63 (the reference
 * cudaHostRegister's one posix_memalign'ed line per flag; here lines are
 * carved out of page-sized cudaHostAlloc'ed slabs so that a thousand flags cost
 * a handful of registrations).
 */
#pragma once
#include <cstdint>

#include "al/cuda/cuda.hpp"
#include "al/util/resource_pool.hpp"

namespace Al {
namespace internal {
namespace cuda {

struct SyncLineFactory {
  int32_t* create();
  void destroy(int32_t*) {}  // slabs are freed together in release_slabs()
  static void release_slabs();
};

extern LockedResourcePool<int32_t*, SyncLineFactory> sync_pool;

}  // namespace cuda
}  // namespace internal
}  // namespace Al
