/**
 * @file profiling.hpp
 * Profiler annotations: named threads and streams, instantaneous marks and
 * nested ranges.
 *
 * Parity: include/aluminum/profiling.hpp:51-74, src/profiling.cpp:43-96.
 * NVTX is resolved at run time (libnvToolsExt is dlopen'ed when present), so
 * the library has no link-time dependency on it and the calls cost one
 * branch when no profiler is attached.
 */
#pragma once
#include <string>

namespace Al {
namespace profiling {

struct ProfileRange {
  unsigned long long id = 0;
  bool active = false;
};

/** Name the calling thread (pthread name and NVTX). */
void name_thread(const std::string& name);
/** Name a CUDA stream for the profiler; `stream` is a cudaStream_t. */
void name_stream(void* stream, const std::string& name);
void mark(const std::string& desc);
ProfileRange prof_start(const std::string& desc);
void prof_end(ProfileRange& r);
/** True when an NVTX implementation was found. */
bool nvtx_available();

/** RAII scope used at every API entry (the role of the reference's Caliper scope macro). */
class Scope {
 public:
  explicit Scope(const char* name);
  ~Scope();
 private:
  ProfileRange r_;
};

}  // namespace profiling
}  // namespace Al

#define AL_API_SCOPE(name) ::Al::profiling::Scope al_api_scope_(name)
