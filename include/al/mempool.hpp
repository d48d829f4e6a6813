/**
 * @file mempool.hpp
 * Process-wide pools of host, pinned-host and device scratch memory.
 * Parity: include/aluminum/mempool.hpp:42-150, src/mempool.cpp:30-34 and the
 * device specialisation at include/aluminum/cuda/cuda_mempool.hpp:46-85.
 * Device memory is served stream-ordered from the CUDA runtime's pool
 * (cudaMallocAsync / cudaFreeAsync) instead of a CUB caching allocator.
 */
#pragma once
#include <cstddef>

#include "al/util/caching_allocator.hpp"

namespace Al {
namespace internal {

class MemoryPool {
 public:
  /** @param stream cudaStream_t for MemoryType::CUDA (stream-ordered), ignored otherwise. */
  void* allocate_bytes(MemoryType mem, size_t bytes, void* stream = nullptr);
  void release_bytes(MemoryType mem, void* ptr, void* stream = nullptr);
  template <MemoryType Mem, typename T>
  T* allocate(size_t n, void* stream = nullptr) {
    return static_cast<T*>(allocate_bytes(Mem, n * sizeof(T), stream));
  }
  template <MemoryType Mem, typename T>
  void release(T* p, void* stream = nullptr) { release_bytes(Mem, p, stream); }
  /** Drop every cached block (called by Finalize while the runtimes are alive). */
  void clear();
};

extern MemoryPool mempool;

}  // namespace internal
}  // namespace Al
