/**
 * @file gpu_status_flag.hpp
 * Device-to-host "event": the stream writes 1 into a pinned word when it
 * reaches the record point; the host polls the word with a plain atomic load.
 * Parity: include/aluminum/cuda/gpu_status_flag.hpp:55-79,
 * src/cuda/gpu_status_flag.cpp:38-98 (cuStreamWriteValue32, cudaEvent fallback).
 */
#pragma once
#include <atomic>
#include <cstdint>

#include "al/cuda/cuda.hpp"

namespace Al {
namespace internal {
namespace cuda {

class GPUStatusFlag {
 public:
  GPUStatusFlag();
  ~GPUStatusFlag();
  GPUStatusFlag(const GPUStatusFlag&) = delete;
  GPUStatusFlag& operator=(const GPUStatusFlag&) = delete;
  /** Clear the flag and enqueue the write of 1 on `stream`. */
  void record(cudaStream_t stream);
  /** Host-side, non-blocking: has the stream passed the record point? */
  bool query();

 private:
  bool use_memops_;
  int32_t* host_flag_ = nullptr;
  CUdeviceptr dev_ptr_ = 0;
  cudaEvent_t event_ = nullptr;
};

}  // namespace cuda
}  // namespace internal
}  // namespace Al
