// Prints whether stream memory operations (cuStreamWriteValue32 / cuStreamWaitValue32) are usable.
// Parity: test/test_stream_mem_ops.cpp:31-41.
#include <iostream>

#include "Al.hpp"
#include "al/cuda/cuda.hpp"

int main() {
  if (!Al::internal::cuda::device_usable()) {
    std::cout << "no CUDA device usable\n";
    return 0;
  }
  Al::Initialize();
  std::cout << "stream memory operations "
            << (Al::internal::cuda::stream_memory_operations_supported() ? "supported" : "not supported") << "\n";
  Al::Finalize();
  return 0;
}
