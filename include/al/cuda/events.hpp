/**
 * @file events.hpp
 * Pool of timing-disabled CUDA events.
 * Parity: include/aluminum/cuda/events.hpp:43-59.
 */
#pragma once
#include "al/cuda/cuda.hpp"
#include "al/util/resource_pool.hpp"

namespace Al {
namespace internal {
namespace cuda {

struct EventFactory {
  cudaEvent_t create() {
    cudaEvent_t e;
    AL_CHECK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    return e;
  }
  void destroy(cudaEvent_t e) { AL_WARN_CUDA(cudaEventDestroy(e)); }
};

extern LockedResourcePool<cudaEvent_t, EventFactory> event_pool;

}  // namespace cuda
}  // namespace internal
}  // namespace Al
