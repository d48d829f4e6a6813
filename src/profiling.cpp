// Profiler hooks with NVTX resolved at run time (see al/profiling.hpp).
#include "al/profiling.hpp"

#include <dlfcn.h>
#include <pthread.h>

#include <atomic>
#include <mutex>

namespace Al {
namespace profiling {

namespace {
// Subset of the NVTX v2 C entry points exported by libnvToolsExt.
using mark_fn = void (*)(const char*);
using range_start_fn = unsigned long long (*)(const char*);
using range_end_fn = void (*)(unsigned long long);
using name_thread_fn = void (*)(unsigned int, const char*);
using name_stream_fn = void (*)(void*, const char*);

struct Nvtx {
  mark_fn mark = nullptr;
  range_start_fn range_start = nullptr;
  range_end_fn range_end = nullptr;
  name_thread_fn name_thread = nullptr;
  name_stream_fn name_stream = nullptr;
  bool ok = false;
};

Nvtx& nvtx() {
  static Nvtx n = [] {
    Nvtx x;
    if (getenv("AL_DISABLE_NVTX")) return x;
    void* h = dlopen("libnvToolsExt.so.1", RTLD_LAZY | RTLD_LOCAL);
    if (!h) h = dlopen("libnvToolsExt.so", RTLD_LAZY | RTLD_LOCAL);
    if (!h) return x;
    x.mark = (mark_fn)dlsym(h, "nvtxMarkA");
    x.range_start = (range_start_fn)dlsym(h, "nvtxRangeStartA");
    x.range_end = (range_end_fn)dlsym(h, "nvtxRangeEnd");
    x.name_thread = (name_thread_fn)dlsym(h, "nvtxNameOsThreadA");
    x.name_stream = (name_stream_fn)dlsym(h, "nvtxNameCudaStreamA");
    x.ok = x.mark && x.range_start && x.range_end;
    return x;
  }();
  return n;
}
}  // namespace

bool nvtx_available() { return nvtx().ok; }

void name_thread(const std::string& name) {
  // pthread names are limited to 15 characters + NUL.
  pthread_setname_np(pthread_self(), name.substr(0, 15).c_str());
  auto& n = nvtx();
  if (n.ok && n.name_thread) n.name_thread((unsigned int)pthread_self(), name.c_str());
}
void name_stream(void* stream, const std::string& name) {
  auto& n = nvtx();
  if (n.ok && n.name_stream) n.name_stream(stream, name.c_str());
}
void mark(const std::string& desc) {
  auto& n = nvtx();
  if (n.ok) n.mark(desc.c_str());
}
ProfileRange prof_start(const std::string& desc) {
  ProfileRange r;
  auto& n = nvtx();
  if (n.ok) {
    r.id = n.range_start(desc.c_str());
    r.active = true;
  }
  return r;
}
void prof_end(ProfileRange& r) {
  if (r.active) {
    nvtx().range_end(r.id);
    r.active = false;
  }
}
Scope::Scope(const char* name) {
  if (nvtx().ok) r_ = prof_start(name);
}
Scope::~Scope() { prof_end(r_); }

}  // namespace profiling
}  // namespace Al
