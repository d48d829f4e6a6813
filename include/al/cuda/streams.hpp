/**
 * @file streams.hpp
 * Pool of internal CUDA streams used by non-blocking operations.
 * Parity: include/aluminum/cuda/streams.hpp:55-99, src/cuda/streams.cpp:41-119
 * (N default-priority + N highest-priority non-blocking streams, round-robin
 * hand-out, replace_streams() to inject application streams, profiler names
 * al_internal_<i> / al_internal_high_<i>).  The default pool size is 4 rather
 * than 1 so that non-blocking operations of different communicators can
 * overlap each other, not only the application's compute stream.
 */
#pragma once
#include <atomic>
#include <functional>
#include <vector>

#include "al/cuda/cuda.hpp"

namespace Al {
namespace internal {
namespace cuda {

class StreamPool {
 public:
  StreamPool() = default;
  ~StreamPool() { /* clear() is called from cuda::finalize while the runtime is alive */ }
  void allocate(size_t num_streams);
  void clear();
  cudaStream_t get_stream();
  cudaStream_t get_high_priority_stream();
  /** Replace every pooled stream with streams supplied by the application; the pool will not destroy them. */
  void replace_streams(std::function<cudaStream_t(bool high_priority)> getter);
  size_t size() const { return default_.size(); }

 private:
  std::vector<cudaStream_t> default_, high_;
  std::atomic<size_t> next_default_{0}, next_high_{0};
  bool external_ = false;
};

extern StreamPool stream_pool;

}  // namespace cuda
}  // namespace internal
}  // namespace Al
