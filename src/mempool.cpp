// Host / pinned / device scratch pools (see al/mempool.hpp).
#include "al/mempool.hpp"

#include <cstdlib>

#include "al/cuda/cuda.hpp"

namespace Al {
namespace internal {

namespace {
struct HostRaw {
  void* allocate(size_t bytes) {
    void* p = nullptr;
    if (posix_memalign(&p, 64, bytes) != 0) throw_al_exception("host allocation of ", bytes, " bytes failed");
    return p;
  }
  void deallocate(void* p, size_t) { free(p); }
};
struct PinnedRaw {
  void* allocate(size_t bytes) {
    void* p = nullptr;
    AL_CHECK_CUDA(cudaMallocHost(&p, bytes));
    return p;
  }
  void deallocate(void* p, size_t) { AL_WARN_CUDA(cudaFreeHost(p)); }
};
CachingAllocator<HostRaw>& host_pool() { static CachingAllocator<HostRaw> a; return a; }
CachingAllocator<PinnedRaw>& pinned_pool() { static CachingAllocator<PinnedRaw> a; return a; }
}  // namespace

MemoryPool mempool;

void* MemoryPool::allocate_bytes(MemoryType mem, size_t bytes, void* stream) {
  switch (mem) {
    case MemoryType::HOST: return host_pool().allocate(bytes);
    case MemoryType::CUDA_PINNED_HOST: return pinned_pool().allocate(bytes);
    case MemoryType::CUDA: {
      void* p = nullptr;
      AL_CHECK_CUDA(cudaMallocAsync(&p, bytes ? bytes : 1, (cudaStream_t)stream));
      return p;
    }
  }
  return nullptr;
}

void MemoryPool::release_bytes(MemoryType mem, void* ptr, void* stream) {
  if (!ptr) return;
  switch (mem) {
    case MemoryType::HOST: host_pool().release(ptr); break;
    case MemoryType::CUDA_PINNED_HOST: pinned_pool().release(ptr); break;
    case MemoryType::CUDA: AL_CHECK_CUDA(cudaFreeAsync(ptr, (cudaStream_t)stream)); break;
  }
}

void MemoryPool::clear() {
  host_pool().clear();
  if (cuda::device_usable()) pinned_pool().clear();
}

}  // namespace internal
}  // namespace Al
