/**
 * @file helper_kernels.hpp
 * Tiny utility kernels: bounded spin-wait on a host-visible word and a fixed
 * delay (used by the event / wait micro-benchmarks).
 * Parity: include/aluminum/cuda/helper_kernels.hpp:37-47,
 * src/cuda/helper_kernels.cu:42-70, benchmark/wait.cu:38-46.
 */
#pragma once
#include <cstdint>

#include "al/cuda/cuda.hpp"

namespace Al {
namespace internal {
namespace cuda {

/**
 * Launch a one-thread kernel that polls `wait_mem` (device-visible) until it
 * equals `wait_value` or `timeout_ns` elapsed; on time-out it stores 1 into
 * `*status` (device-visible, may be null) and returns.
 */
void launch_wait_kernel(cudaStream_t stream, int32_t wait_value, volatile int32_t* wait_mem,
                        uint64_t timeout_ns, int32_t* status);
/** Stream-memory-operation flavour: cuStreamWaitValue32(stream, wait_mem, wait_value, EQ). */
void launch_wait_kernel(cudaStream_t stream, int32_t wait_value, CUdeviceptr wait_mem);
/** Occupy `stream` for about `nanoseconds`. */
void launch_delay_kernel(cudaStream_t stream, uint64_t nanoseconds);

}  // namespace cuda
}  // namespace internal
}  // namespace Al
