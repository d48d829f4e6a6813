/**
 * @file resource_pool.hpp
 * Mutex-guarded stack of interchangeable resources (events, pinned flag lines).
 * Parity: include/aluminum/utils/locked_resource_pool.hpp:50-102
 * (preallocate / get / release / clear).
 */
#pragma once
#include <mutex>
#include <vector>

namespace Al {
namespace internal {

/**
 * @tparam Res     handle type (cheap to copy)
 * @tparam Factory has `Res create()` and `void destroy(Res)`
 */
template <typename Res, typename Factory>
class LockedResourcePool {
 public:
  LockedResourcePool() = default;
  explicit LockedResourcePool(Factory f) : factory_(std::move(f)) {}
  ~LockedResourcePool() { /* resources are destroyed by an explicit clear() */ }

  void preallocate(size_t n) {
    std::lock_guard<std::mutex> g(mu_);
    for (size_t i = 0; i < n; ++i) free_.push_back(factory_.create());
  }
  Res get() {
    {
      std::lock_guard<std::mutex> g(mu_);
      if (!free_.empty()) {
        Res r = free_.back();
        free_.pop_back();
        return r;
      }
    }
    return factory_.create();
  }
  void release(Res r) {
    std::lock_guard<std::mutex> g(mu_);
    free_.push_back(r);
  }
  void clear() {
    std::lock_guard<std::mutex> g(mu_);
    for (auto& r : free_) factory_.destroy(r);
    free_.clear();
  }
  size_t idle() {
    std::lock_guard<std::mutex> g(mu_);
    return free_.size();
  }

 private:
  std::mutex mu_;
  std::vector<Res> free_;
  Factory factory_;
};

}  // namespace internal
}  // namespace Al
