// Shared helpers of the C++ test and benchmark programs: deterministic data
// that any rank can regenerate for any other rank (so a serial oracle needs no
// communication), typed buffers living on the host or the device depending on
// the backend, argument parsing, size sweeps and a hang watchdog.
//
// Parity: test/test_utils.hpp:157-651 (data generation, VectorType, size
// sweeps, check_vector), test/cuda_vector.hpp:36-167, test/hang_watchdog.hpp:43-140.
#pragma once
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <iostream>
#include <map>
#include <mutex>
#include <random>
#include <string>
#include <thread>
#include <vector>

#include "Al.hpp"
#include "al/host/reduce.hpp"

namespace altest {

// ---- 16-bit float wrappers usable as element types -------------------------
using half_t = Al::half_t;
using bf16_t = Al::bfloat16_t;

template <typename T> inline double to_double(T v) { return (double)v; }
template <> inline double to_double<half_t>(half_t v) { return Al::internal::host::half_to_float(v.bits); }
template <> inline double to_double<bf16_t>(bf16_t v) { return Al::internal::host::bf16_to_float(v.bits); }
template <typename T> inline T from_double(double d) { return (T)d; }
template <> inline half_t from_double<half_t>(double d) { return half_t{Al::internal::host::float_to_half((float)d)}; }
template <> inline bf16_t from_double<bf16_t>(double d) { return bf16_t{Al::internal::host::float_to_bf16((float)d)}; }

template <typename T> struct is_float_like : std::is_floating_point<T> {};
template <> struct is_float_like<half_t> : std::true_type {};
template <> struct is_float_like<bf16_t> : std::true_type {};

/**
 * Deterministic input of `rank`: element i of stream `tag`.  Values are small
 * multiples of 1/8 (floats) or small integers, so sums over up to 8 ranks are
 * exact even in bfloat16; for products the values are +-1.
 */
template <typename T>
std::vector<T> gen_data(size_t n, int rank, Al::ReductionOperator op, unsigned tag = 0) {
  std::minstd_rand rng((unsigned)(rank + 1) * 7919u + tag * 104729u + 17u);
  std::vector<T> v(n);
  const bool prod = op == Al::ReductionOperator::prod;
  for (size_t i = 0; i < n; ++i) {
    const unsigned r = (unsigned)rng();
    if (prod) v[i] = from_double<T>((r & 1) ? 1.0 : (std::is_unsigned<T>::value ? 1.0 : -1.0));
    else if (is_float_like<T>::value) v[i] = from_double<T>(((int)(r % 33) - 16) / 8.0);
    else if (std::is_unsigned<T>::value) v[i] = from_double<T>((double)(r % 13));
    else v[i] = from_double<T>((double)((int)(r % 13) - 6));
  }
  return v;
}

/** Serial oracle: fold the given vectors element-wise in rank order. */
template <typename T>
std::vector<T> reduce_oracle(const std::vector<std::vector<T>>& ins, Al::ReductionOperator op) {
  const size_t n = ins[0].size();
  std::vector<T> out(n);
  std::vector<const void*> srcs;
  for (auto& v : ins) srcs.push_back(v.data());
  if (n) Al::internal::host::reduce_multi(Al::TypeMap<T>::value, op, out.data(), srcs.data(), (int)srcs.size(), n);
  return out;
}

template <typename T>
bool check_vector(const std::vector<T>& got, const std::vector<T>& want, const char* what, int rank, double eps = 1e-4) {
  if (got.size() != want.size()) {
    fprintf(stderr, "[rank %d] %s: size %zu != %zu\n", rank, what, got.size(), want.size());
    return false;
  }
  for (size_t i = 0; i < got.size(); ++i) {
    const double g = to_double(got[i]), w = to_double(want[i]);
    const double tol = is_float_like<T>::value ? eps * (1.0 + std::fabs(w)) : 0.0;
    if (!(std::fabs(g - w) <= tol)) {
      fprintf(stderr, "[rank %d] %s: mismatch at %zu of %zu: got %.9g want %.9g\n", rank, what, i, got.size(), g, w);
      return false;
    }
  }
  return true;
}

// ---- buffers -----------------------------------------------------------------
/** Host backend: plain vector. */
template <typename Backend, typename T>
struct Buffer {
  std::vector<T> v;
  explicit Buffer(size_t n = 0) : v(n) {}
  T* data() { return v.empty() ? nullptr : v.data(); }
  size_t size() const { return v.size(); }
  void upload(const std::vector<T>& h, typename Backend::comm_type&) { v = h; }
  std::vector<T> download(typename Backend::comm_type&) { return v; }
};

#ifdef AL_HAS_CUDA
/**
 * Device memory of the test buffers.  Blocks go back to a process-wide free list instead of cudaFree:
 * cudaFree synchronises the whole device, and with several threads testing at once (--threads) that means
 * waiting for another thread's collective, which in turn waits for a peer rank whose thread sits in the same
 * cudaFree - every rank stuck.  (The reference's test vectors come from its caching pool for the same
 * reason, test/cuda_vector.hpp:36-167.)  The list is released at process exit.
 */
class DevicePool {
 public:
  static DevicePool& get() { static DevicePool* p = new DevicePool; return *p; }
  void* take(size_t bytes) {
    const size_t key = round(bytes);
    {
      std::lock_guard<std::mutex> lock(mu_);
      auto it = free_.find(key);
      if (it != free_.end() && !it->second.empty()) {
        void* p = it->second.back();
        it->second.pop_back();
        return p;
      }
    }
    void* p = nullptr;
    AL_CHECK_CUDA(cudaMalloc(&p, key));
    return p;
  }
  void give(void* p, size_t bytes) {
    std::lock_guard<std::mutex> lock(mu_);
    free_[round(bytes)].push_back(p);
  }

 private:
  static size_t round(size_t b) { size_t r = 256; while (r < b) r <<= 1; return r; }
  std::mutex mu_;
  std::map<size_t, std::vector<void*>> free_;
};

template <typename T>
struct DeviceBuf {
  T* p = nullptr;
  size_t n = 0;
  explicit DeviceBuf(size_t n_ = 0) : n(n_) {
    if (n) p = (T*)DevicePool::get().take(n * sizeof(T));
  }
  ~DeviceBuf() { if (p) DevicePool::get().give(p, n * sizeof(T)); }
  DeviceBuf(const DeviceBuf&) = delete;
  DeviceBuf& operator=(const DeviceBuf&) = delete;
  DeviceBuf(DeviceBuf&& o) noexcept : p(o.p), n(o.n) { o.p = nullptr; o.n = 0; }
  T* data() { return p; }
  size_t size() const { return n; }
  void upload_on(const std::vector<T>& h, cudaStream_t s) {
    if (h.size() != n) throw_al_exception("upload size mismatch");
    if (n) AL_CHECK_CUDA(cudaMemcpyAsync(p, h.data(), n * sizeof(T), cudaMemcpyHostToDevice, s));
    AL_CHECK_CUDA(cudaStreamSynchronize(s));
  }
  std::vector<T> download_on(cudaStream_t s) {
    std::vector<T> h(n);
    AL_CHECK_CUDA(cudaStreamSynchronize(s));
    if (n) AL_CHECK_CUDA(cudaMemcpy(h.data(), p, n * sizeof(T), cudaMemcpyDeviceToHost));
    return h;
  }
};
template <typename T>
struct Buffer<Al::DeviceBackend, T> : DeviceBuf<T> {
  using DeviceBuf<T>::DeviceBuf;
  void upload(const std::vector<T>& h, Al::DeviceCommunicator& c) { this->upload_on(h, c.get_stream()); }
  std::vector<T> download(Al::DeviceCommunicator& c) { return this->download_on(c.get_stream()); }
};
template <typename T>
struct Buffer<Al::HostTransferBackend, T> : DeviceBuf<T> {
  using DeviceBuf<T>::DeviceBuf;
  void upload(const std::vector<T>& h, Al::HostTransferCommunicator& c) { this->upload_on(h, c.get_stream()); }
  std::vector<T> download(Al::HostTransferCommunicator& c) { return this->download_on(c.get_stream()); }
};
#endif

// ---- options -------------------------------------------------------------------
struct Args {
  std::map<std::string, std::string> kv;
  Args(int argc, char** argv) {
    for (int i = 1; i < argc; ++i) {
      std::string a = argv[i];
      if (a.rfind("--", 0) != 0) continue;
      a = a.substr(2);
      if (i + 1 < argc && std::string(argv[i + 1]).rfind("--", 0) != 0) kv[a] = argv[++i];
      else kv[a] = "1";
    }
  }
  bool has(const std::string& k) const { return kv.count(k) != 0; }
  std::string str(const std::string& k, const std::string& d) const { auto it = kv.find(k); return it == kv.end() ? d : it->second; }
  long num(const std::string& k, long d) const { auto it = kv.find(k); return it == kv.end() ? d : atol(it->second.c_str()); }
};

inline Al::ReductionOperator parse_redop(const std::string& s) {
  static const std::map<std::string, Al::ReductionOperator> m = {
      {"sum", Al::ReductionOperator::sum}, {"prod", Al::ReductionOperator::prod}, {"min", Al::ReductionOperator::min},
      {"max", Al::ReductionOperator::max}, {"lor", Al::ReductionOperator::lor}, {"land", Al::ReductionOperator::land},
      {"lxor", Al::ReductionOperator::lxor}, {"bor", Al::ReductionOperator::bor}, {"band", Al::ReductionOperator::band},
      {"bxor", Al::ReductionOperator::bxor}, {"avg", Al::ReductionOperator::avg}};
  auto it = m.find(s);
  if (it == m.end()) throw_al_exception("unknown reduction operator ", s);
  return it->second;
}

/** Powers of two in [lo, hi], optionally each followed by size+1, optionally 0 first. */
inline std::vector<size_t> sweep_sizes(size_t lo, size_t hi, bool odd, bool zero) {
  std::vector<size_t> s;
  if (zero) s.push_back(0);
  for (size_t n = lo ? lo : 1; n <= hi; n *= 2) {
    s.push_back(n);
    if (odd) s.push_back(n + 1);
  }
  return s;
}

/** Aborts the process when an armed section does not finish in time. */
class HangWatchdog {
 public:
  explicit HangWatchdog(double seconds) : limit_(seconds), th_([this] { loop(); }) {}
  ~HangWatchdog() { stop_ = true; th_.join(); }
  void arm(const std::string& what) {
    std::lock_guard<std::mutex> g(m_);
    what_ = what;
    t0_ = now();
    armed_ = true;
  }
  void disarm() { armed_ = false; }
 private:
  static double now() { return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count(); }
  void loop() {
    while (!stop_) {
      std::unique_lock<std::mutex> g(m_);
      if (armed_ && now() - t0_ > limit_) {
        fprintf(stderr, "hang watchdog: '%s' exceeded %.0f s, aborting\n", what_.c_str(), limit_);
        fflush(stderr);
        _exit(86);
      }
      g.unlock();
      std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
  }
  double limit_;
  std::atomic<bool> stop_{false}, armed_{false};
  std::mutex m_;
  std::string what_;
  double t0_ = 0;
  std::thread th_;
};

}  // namespace altest
