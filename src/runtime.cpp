// Library life cycle: Initialize / Finalize, the fatal-signal handler and the
// process-wide singletons (see al/runtime.hpp).
#include "al/runtime.hpp"

#include <execinfo.h>
#include <signal.h>
#include <unistd.h>

#include <fstream>
#include <iostream>
#include <mutex>

#include "al/cuda/cuda.hpp"
#include "al/mempool.hpp"
#include "al/trace.hpp"
#include "al/tuning.hpp"

namespace Al {

namespace {

struct Runtime {
  std::unique_ptr<internal::World> world;
  std::unique_ptr<internal::ProgressEngine> pe;
  bool cuda_on = false;
  bool handlers_installed = false;
};

Runtime* g_rt = nullptr;
std::mutex g_mu;

const int kSignals[] = {SIGILL, SIGABRT, SIGFPE, SIGBUS, SIGSEGV};
struct sigaction g_old[5];

// Post-mortem: backtrace + progress-engine state into "<host>.<pid>.dump.txt",
// then the trace, then re-raise with the previous disposition.
void fatal_handler(int sig) {
  static volatile sig_atomic_t entered = 0;
  if (!entered) {
    entered = 1;
    char host[256] = "localhost";
    gethostname(host, sizeof(host) - 1);
    std::string path = internal::env_str("AL_TRACE_DIR", ".") + "/" + host + "." + std::to_string(getpid()) + ".dump.txt";
    std::ofstream f(path);
    if (f) {
      f << "Fatal signal " << sig << "\nBacktrace:\n";
      void* frames[64];
      int n = backtrace(frames, 64);
      char** syms = backtrace_symbols(frames, n);
      for (int i = 0; i < n; ++i) f << "  " << (syms ? syms[i] : "?") << "\n";
      if (g_rt && g_rt->pe) g_rt->pe->dump_state(f);
      f.flush();
    }
    trace::write_to_file();
  }
  for (int i = 0; i < 5; ++i)
    if (kSignals[i] == sig) sigaction(sig, &g_old[i], nullptr);
  raise(sig);
}

void install_handlers(Runtime& rt) {
  if (!tuning().signal_handler) return;
  struct sigaction sa;
  memset(&sa, 0, sizeof(sa));
  sa.sa_handler = fatal_handler;
  sigemptyset(&sa.sa_mask);
  for (int i = 0; i < 5; ++i) sigaction(kSignals[i], &sa, &g_old[i]);
  rt.handlers_installed = true;
}

void remove_handlers(Runtime& rt) {
  if (!rt.handlers_installed) return;
  for (int i = 0; i < 5; ++i) sigaction(kSignals[i], &g_old[i], nullptr);
  rt.handlers_installed = false;
}

}  // namespace

void Initialize() {
  std::lock_guard<std::mutex> g(g_mu);
  if (g_rt) return;
  tuning().load_from_env();
  trace::enable(tuning().trace);
  std::unique_ptr<Runtime> rt(new Runtime());
  rt->world = internal::World::from_env();
  rt->pe.reset(new internal::ProgressEngine());
  if (internal::cuda::device_usable()) {
    // One process drives one GPU: pick it from the node-local rank unless the
    // application (or AL_GPU_ID) already chose.
    int ndev = 0;
    AL_CHECK_CUDA(cudaGetDeviceCount(&ndev));
    long forced = internal::env_long("AL_GPU_ID", -1);
    if (forced >= 0) AL_CHECK_CUDA(cudaSetDevice((int)(forced % ndev)));
    else if (internal::env_long("AL_SET_DEVICE", 1) != 0 && rt->world->size() > 1)
      AL_CHECK_CUDA(cudaSetDevice(rt->world->local_rank() % ndev));
    int dev = 0;
    AL_CHECK_CUDA(cudaGetDevice(&dev));
    rt->pe->set_device(dev);
    internal::cuda::init();
    rt->cuda_on = true;
  }
  if (!tuning().pe_start_on_demand) rt->pe->run();
  install_handlers(*rt);
  g_rt = rt.release();
}

void Initialize(int& /*argc*/, char**& /*argv*/) { Initialize(); }

void Finalize() {
  std::lock_guard<std::mutex> g(g_mu);
  if (!g_rt) return;
  remove_handlers(*g_rt);
  g_rt->pe->stop();
  if (g_rt->cuda_on) {
    (void)cudaDeviceSynchronize();
    internal::mempool.clear();
    internal::cuda::finalize();
  } else {
    internal::mempool.clear();
  }
  g_rt->pe.reset();
  g_rt->world.reset();
  trace::write_to_file();
  delete g_rt;
  g_rt = nullptr;
}

bool Initialized() {
  std::lock_guard<std::mutex> g(g_mu);
  return g_rt != nullptr;
}

std::vector<int> AliveRanks() {
  internal::World* w = internal::get_world();
  std::vector<int> alive;
  for (int r = 0; r < w->size(); ++r)
    if (w->peer_alive(r)) alive.push_back(r);
  return alive;
}

namespace internal {

ProgressEngine* get_progress_engine() {
  if (!g_rt) throw_al_exception("the library is not initialised (call Al::Initialize first)");
  return g_rt->pe.get();
}

ProgressEngine* get_progress_engine_if_any() { return g_rt ? g_rt->pe.get() : nullptr; }

void release_progress_key(const void* key) {
  if (g_rt && g_rt->pe) g_rt->pe->release_key(key);
}

World* get_world() {
  if (!g_rt) throw_al_exception("the library is not initialised (call Al::Initialize first)");
  return g_rt->world.get();
}

bool cuda_available() { return g_rt && g_rt->cuda_on; }

}  // namespace internal
}  // namespace Al
