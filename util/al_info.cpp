// al_info - prints version, compiled features, the tuning table and, when a
// GPU is usable, the discovered topology.  Parity: util/al_info.cpp:34-95.
#include <iostream>

#include "Al.hpp"
#include "al/cuda/cuda.hpp"
#include "al/device/symmem.hpp"
#include "al/progress.hpp"
#include "al/tuning.hpp"

int main() {
  std::cout << "Aluminum-B200 " << AL_VERSION << "\n";
  std::cout << "Backends: host";
#ifdef AL_HAS_CUDA
  std::cout << " device host-transfer rma";
#endif
  std::cout << "\nFeatures:"
            << " thread_multiple=1 trace=runtime(AL_TRACE) debug_checks=runtime(AL_DEBUG)"
            << " nvtx=" << (Al::profiling::nvtx_available() ? "found" : "not-found")
            << " half=1 bfloat16=1\n";
  std::cout << "Kernel target: sm_100a, max device ranks " << AL_MAX_DEVICE_RANKS << "\n";
  std::cout << "--- tuning ---\n" << Al::tuning().describe();
#ifdef AL_HAS_CUDA
  std::cout << "--- topology ---\n";
  if (Al::internal::cuda::device_usable()) {
    std::cout << Al::internal::device::discover_topology().describe();
    Al::Initialize();
    std::cout << "stream memory operations: "
              << (Al::internal::cuda::stream_memory_operations_supported() ? "supported" : "unsupported") << "\n";
    Al::Finalize();
  } else {
    std::cout << "no CUDA device usable in this process\n";
  }
#endif
  // Where the progress thread of this process polls from (a core local to the GPU when the kernel tells which those are).
  std::cout << "--- progress thread ---\n";
  Al::Initialize();
  {
    Al::internal::ProgressEngine* pe = Al::internal::get_progress_engine();
    pe->run();  // started on demand otherwise; run() returns once the thread has bound itself
    std::cout << "bound to core " << pe->bound_core() << " (-1: not bound), cores reported local to the GPU: "
              << pe->near_gpu_cores() << "\n";
  }
  Al::Finalize();
  return 0;
}
