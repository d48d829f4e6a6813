/**
 * @file gpu_wait.hpp
 * Host-to-device gate: a stream stalls at wait() until the host calls signal().
 * Parity: include/aluminum/cuda/gpu_wait.hpp:56-74, src/cuda/gpu_wait.cpp:38-74
 * (cuStreamWaitValue32 on a pinned word, spin-kernel fallback).  The fallback
 * kernel here is bounded: it gives up after a time budget and reports through
 * a status word instead of spinning forever.
 */
#pragma once
#include <cstdint>

#include "al/cuda/cuda.hpp"

namespace Al {
namespace internal {
namespace cuda {

class GPUWait {
 public:
  GPUWait();
  ~GPUWait();
  GPUWait(const GPUWait&) = delete;
  GPUWait& operator=(const GPUWait&) = delete;
  /** Enqueue a wait on `stream` that completes once signal() has been called. */
  void wait(cudaStream_t stream);
  /** Release every stream waiting on this object (host atomic store). */
  void signal();
  /**
   * True once a wait of the spin-kernel fallback has given up (its time budget ran out before signal()): the
   * stream has gone on without the host, so whatever it produced afterwards must not be trusted.  Always false
   * where stream memory operations do the waiting (they have no time budget).
   */
  bool timed_out() const;

 private:
  int32_t* host_flag_ = nullptr;
  int32_t* host_status_ = nullptr;  ///< pinned word the fallback kernel sets when it gives up
  CUdeviceptr dev_ptr_ = 0;
};

}  // namespace cuda
}  // namespace internal
}  // namespace Al
