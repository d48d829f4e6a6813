// Utility kernels of the CUDA support layer (see al/cuda/helper_kernels.hpp).
#include "al/cuda/helper_kernels.hpp"

namespace Al {
namespace internal {
namespace cuda {

namespace {

__device__ __forceinline__ uint64_t global_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__global__ void bounded_spin_wait_kernel(int32_t wait_value, volatile int32_t* wait_mem,
                                         uint64_t timeout_ns, int32_t* status) {
  const uint64_t t0 = global_ns();
  for (;;) {
    if (*wait_mem == wait_value) return;
    __nanosleep(200);
    if (global_ns() - t0 > timeout_ns) {
      if (status) {
        *status = 1;
        __threadfence_system();
      }
      return;
    }
  }
}

__global__ void delay_kernel(uint64_t ns) {
  const uint64_t t0 = global_ns();
  while (global_ns() - t0 < ns) __nanosleep(100);
}

}  // namespace

void launch_wait_kernel(cudaStream_t stream, int32_t wait_value, volatile int32_t* wait_mem,
                        uint64_t timeout_ns, int32_t* status) {
  bounded_spin_wait_kernel<<<1, 1, 0, stream>>>(wait_value, wait_mem, timeout_ns, status);
  AL_CHECK_CUDA(cudaGetLastError());
}

void launch_wait_kernel(cudaStream_t stream, int32_t wait_value, CUdeviceptr wait_mem) {
  const auto& d = drv();
  if (!d.StreamWaitValue32) throw_al_exception("stream memory operations are not available");
  AL_CHECK_CUDA_DRV(d.StreamWaitValue32((CUstream)stream, wait_mem, (cuuint32_t)wait_value,
                                        CU_STREAM_WAIT_VALUE_EQ));
}

void launch_delay_kernel(cudaStream_t stream, uint64_t nanoseconds) {
  // Cap the delay: this kernel exists for micro-benchmarks, never to park a GPU.
  if (nanoseconds > 2000000000ull) nanoseconds = 2000000000ull;
  delay_kernel<<<1, 1, 0, stream>>>(nanoseconds);
  AL_CHECK_CUDA(cudaGetLastError());
}

}  // namespace cuda
}  // namespace internal
}  // namespace Al
