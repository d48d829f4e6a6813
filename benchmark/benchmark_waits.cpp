// benchmark_waits - cost of gating a stream on a host-written flag: the stream-memory-operation
// wait (cuStreamWaitValue32) against the bounded spin kernel, measured as (a) host time to enqueue
// the wait and (b) time from the host's signal to the stream passing the gate.
// Parity: benchmark/benchmark_waits.cpp:71-108 of the reference.
#include <cstdio>

#include "Al.hpp"
#include "al/cuda/gpu_status_flag.hpp"
#include "al/cuda/gpu_wait.hpp"
#include "al/cuda/helper_kernels.hpp"
#include "al/cuda/sync_memory.hpp"

using namespace Al::internal::cuda;

int main(int argc, char** argv) {
  const int iters = argc > 1 ? atoi(argv[1]) : 2000;
  Al::Initialize();
  if (!device_usable()) { printf("no CUDA device\n"); return 0; }
  cudaStream_t s;
  AL_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  for (int mode = 0; mode < 2; ++mode) {
    if (mode == 0 && !stream_memory_operations_supported()) continue;
    double enqueue = 0, release = 0;
    int32_t* flag = sync_pool.get();
    void* dp = nullptr;
    AL_CHECK_CUDA(cudaHostGetDevicePointer(&dp, flag, 0));
    for (int i = 0; i < iters; ++i) {
      __atomic_store_n(flag, 0, __ATOMIC_SEQ_CST);
      GPUStatusFlag passed;
      double t0 = Al::get_time();
      if (mode == 0) launch_wait_kernel(s, 1, (CUdeviceptr)dp);
      else launch_wait_kernel(s, 1, (volatile int32_t*)dp, 1000000000ull, nullptr);
      enqueue += Al::get_time() - t0;
      passed.record(s);
      t0 = Al::get_time();
      __atomic_store_n(flag, 1, __ATOMIC_SEQ_CST);
      while (!passed.query()) {}
      release += Al::get_time() - t0;
    }
    sync_pool.release(flag);
    printf("%-28s enqueue %.2f us   signal-to-pass %.2f us\n", mode == 0 ? "stream memory operation" : "bounded spin kernel",
           enqueue / iters * 1e6, release / iters * 1e6);
  }
  AL_CHECK_CUDA(cudaStreamDestroy(s));
  Al::Finalize();
  return 0;
}
