/**
 * @file utils.hpp
 * Small helpers: steady-clock time in seconds and an exclusive prefix sum.
 * Parity: include/aluminum/utils/utils.hpp:36-54.
 */
#pragma once
#include <chrono>
#include <cstdlib>
#include <string>
#include <vector>

namespace Al {

/** Seconds since an arbitrary fixed point (monotonic). */
inline double get_time() {
  using namespace std::chrono;
  return duration_cast<duration<double>>(steady_clock::now().time_since_epoch()).count();
}

/** out[i] = sum of in[0..i). */
template <typename T>
std::vector<T> excl_prefix_sum(const std::vector<T>& in) {
  std::vector<T> out(in.size());
  T run{};
  for (size_t i = 0; i < in.size(); ++i) { out[i] = run; run += in[i]; }
  return out;
}

namespace internal {
inline long env_long(const char* name, long dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  long r = std::strtol(v, &end, 0);
  return end == v ? dflt : r;
}
/** Fractions allowed ("0.5"); unparsable text gives the default. */
inline double env_double(const char* name, double dflt) {
  const char* v = std::getenv(name);
  if (!v || !*v) return dflt;
  char* end = nullptr;
  double r = std::strtod(v, &end);
  return end == v ? dflt : r;
}
inline std::string env_str(const char* name, const std::string& dflt = "") {
  const char* v = std::getenv(name);
  return (v && *v) ? std::string(v) : dflt;
}
}  // namespace internal
}  // namespace Al
