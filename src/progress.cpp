// The progress engine thread (see al/progress.hpp for the contract).
#include "al/progress.hpp"

#include <fstream>
#include <algorithm>
#include <memory>

#include <pthread.h>
#include <sched.h>

#include <algorithm>
#include <iostream>
#include <sstream>

#include "al/base.hpp"
#include "al/trace.hpp"
#include "al/tuning.hpp"
#include "al/util/utils.hpp"

#if defined(__x86_64__)
#include <immintrin.h>
#define AL_CPU_RELAX() _mm_pause()
#else
#define AL_CPU_RELAX() ((void)0)
#endif

namespace Al {
namespace internal {

// Implemented by the CUDA layer; a weak no-op keeps host-only tools linkable.
void pe_make_device_current(int dev);
std::string pe_device_pci_bus_id(int dev);

std::vector<int> parse_cpulist(const std::string& text) {
  // sysfs format: "0-31,64-95" (ranges and single numbers, comma separated)
  std::vector<int> out;
  size_t i = 0;
  auto number = [&](int& v) {
    if (i >= text.size() || !isdigit((unsigned char)text[i])) return false;
    v = 0;
    while (i < text.size() && isdigit((unsigned char)text[i])) v = v * 10 + (text[i++] - '0');
    return true;
  };
  while (i < text.size()) {
    int a = 0, b = 0;
    if (!number(a)) { ++i; continue; }
    b = a;
    if (i < text.size() && text[i] == '-') { ++i; if (!number(b)) b = a; }
    for (int c = a; c <= b && c < CPU_SETSIZE; ++c) out.push_back(c);
  }
  return out;
}

int choose_pe_core(const std::vector<int>& allowed, const std::vector<int>& near_gpu, long local_rank) {
  if (allowed.size() < 2) return -1;  // nothing to gain, and never steal the only core
  // Cores that are both allowed and local to the GPU; all allowed cores when that set is empty.
  std::vector<int> pool;
  for (int c : near_gpu)
    if (std::find(allowed.begin(), allowed.end(), c) != allowed.end()) pool.push_back(c);
  if (pool.empty()) pool = allowed;
  std::sort(pool.begin(), pool.end());
  // The highest-numbered cores are the least likely to run the application's main threads; co-located
  // ranks step down from the top by their node-local rank so that they do not share a core.
  const size_t idx = pool.size() - 1 - (size_t)(local_rank % (long)pool.size());
  return pool[idx];
}

ProgressEngine::ProgressEngine() = default;

ProgressEngine::~ProgressEngine() {
  stop();
  for (size_t i = 0; i < num_queues_.load(); ++i) delete queues_[i];
}

void ProgressEngine::run() {
  std::unique_lock<std::mutex> lk(start_mu_);
  if (started_.load(std::memory_order_acquire)) return;
  if (starting_) {
    // Another caller is bringing the thread up (its wait below released the lock): wait for it.
    start_cv_.wait(lk, [this] { return started_.load(std::memory_order_acquire); });
    return;
  }
  starting_ = true;
  stop_flag_.store(false);
  thread_ready_ = false;
  thread_ = std::thread(&ProgressEngine::engine, this);
  start_cv_.wait(lk, [this] { return thread_ready_; });
  started_.store(true, std::memory_order_release);
  starting_ = false;
  start_cv_.notify_all();
}

void ProgressEngine::stop() {
  std::unique_lock<std::mutex> lk(start_mu_);
  if (!started_.load(std::memory_order_acquire)) return;
  stop_flag_.store(true, std::memory_order_release);
  lk.unlock();
  if (thread_.joinable()) thread_.join();
  lk.lock();
  started_.store(false, std::memory_order_release);
}

namespace {
// Key of a slot whose ordering domain was released; never a valid stream or communicator address.
const void* const kFreeKey = &kFreeKey;
}  // namespace

void ProgressEngine::release_key(const void* key) {
  std::lock_guard<std::mutex> g(add_mu_);
  const size_t n = num_queues_.load(std::memory_order_acquire);
  for (size_t i = 0; i < n; ++i)
    if (queues_[i]->key.load(std::memory_order_relaxed) == key) queues_[i]->key.store(kFreeKey, std::memory_order_release);
}

ProgressEngine::InputQueue* ProgressEngine::queue_for(const void* key) {
  // Fast path: lock-free scan of the published slots.
  size_t n = num_queues_.load(std::memory_order_acquire);
  for (size_t i = 0; i < n; ++i)
    if (queues_[i]->key.load(std::memory_order_acquire) == key) return queues_[i];
  std::lock_guard<std::mutex> g(add_mu_);
  n = num_queues_.load(std::memory_order_acquire);
  for (size_t i = 0; i < n; ++i)
    if (queues_[i]->key.load(std::memory_order_relaxed) == key) return queues_[i];
  for (size_t i = 0; i < n; ++i)
    if (queues_[i]->key.load(std::memory_order_relaxed) == kFreeKey) {  // reuse a released slot
      queues_[i]->key.store(key, std::memory_order_release);
      return queues_[i];
    }
  if (n >= AL_PE_NUM_STREAMS)
    throw_al_exception("progress engine: more than ", AL_PE_NUM_STREAMS,
                       " distinct streams/communicators have outstanding asynchronous work");
  queues_[n] = new InputQueue(key);
  num_queues_.store(n + 1, std::memory_order_release);
  return queues_[n];
}

void ProgressEngine::enqueue(AlState* state) {
  // The engine owns the state from here on, also when it cannot take it.
  std::unique_ptr<AlState> guard(state);
  if (!started_.load(std::memory_order_acquire)) run();
  InputQueue* q = queue_for(state->get_compute_stream());
  if (!q->q.try_push(state))
    throw_al_exception("progress engine input queue overflow (", AL_PE_INPUT_QUEUE_SIZE, " entries)");
  guard.release();
  pending_inputs_.fetch_add(1, std::memory_order_release);
}

void ProgressEngine::set_hang_callback(std::function<void(const AlState&, double)> cb) {
  std::lock_guard<std::mutex> g(cb_mu_);
  hang_cb_ = std::move(cb);
}

std::ostream& ProgressEngine::dump_state(std::ostream& os) {
  // Best effort: reads engine-private queues without synchronisation, which is
  // acceptable for a post-mortem dump.
  const size_t n = num_queues_.load(std::memory_order_acquire);
  os << "Progress engine: " << n << " stream(s), " << in_flight_.load() << " state(s) in flight\n";
  for (size_t i = 0; i < n; ++i) {
    os << " stream " << i << " key=" << queues_[i]->key.load() << "\n";
    for (int s = 0; s < AL_PE_NUM_PIPELINE_STAGES; ++s) {
      os << "  stage " << s << ":";
      for (AlState* st : pipelines_[i].stage[s]) {
        os << " [" << st->get_name() << " " << st->get_desc()
           << (st->paused_for_advance ? " paused" : "") << "]";
      }
      os << "\n";
    }
  }
  return os;
}

void ProgressEngine::bind() {
  if (!tuning().pe_bind_thread) return;
  // The thread polls flags that the GPU writes into pinned host memory and answers with stores the GPU
  // waits for: it belongs on a core of the socket the GPU hangs off (the reference asks hwloc for the
  // GPU's cpuset, src/progress.cpp:394-495; here the kernel's own answer is read from sysfs:
  // /sys/bus/pci/devices/<bus id>/local_cpulist).  AL_PE_CORE pins it to a given core instead.
  cpu_set_t mask;
  CPU_ZERO(&mask);
  if (sched_getaffinity(0, sizeof(mask), &mask) != 0) return;
  std::vector<int> allowed;
  for (int c = 0; c < CPU_SETSIZE; ++c)
    if (CPU_ISSET(c, &mask)) allowed.push_back(c);
  int core = (int)env_long("AL_PE_CORE", -1);
  if (core < 0) {
    std::vector<int> near_gpu;
    const std::string bus = device_ >= 0 ? pe_device_pci_bus_id(device_) : std::string();
    if (!bus.empty()) {
      std::ifstream f("/sys/bus/pci/devices/" + bus + "/local_cpulist");
      std::string line;
      if (f && std::getline(f, line)) near_gpu = parse_cpulist(line);
    }
    near_gpu_cores_ = (int)near_gpu.size();
    core = choose_pe_core(allowed, near_gpu, env_long("AL_LOCAL_RANK", env_long("LOCAL_RANK", 0)));
  }
  if (core < 0) return;
  cpu_set_t one;
  CPU_ZERO(&one);
  CPU_SET(core, &one);
  if (pthread_setaffinity_np(pthread_self(), sizeof(one), &one) == 0) bound_core_ = core;
}

void ProgressEngine::engine() {
  bind();
  if (device_ >= 0) pe_make_device_current(device_);
  profiling::name_thread("al-progress");
  {
    std::lock_guard<std::mutex> lk(start_mu_);
    thread_ready_ = true;
  }
  start_cv_.notify_all();

  unsigned idle_spins = 0;
  while (!stop_flag_.load(std::memory_order_acquire)) {
    const size_t limit = (size_t)std::max(1, tuning().pe_num_concurrent_ops);
    const double hang_s = tuning().pe_hang_seconds;
    // ---- admission ---------------------------------------------------------
    const size_t nq = num_queues_.load(std::memory_order_acquire);
    if (pending_inputs_.load(std::memory_order_acquire) > 0) {
      for (size_t i = 0; i < nq; ++i) {
        AlState* st = nullptr;
        while (queues_[i]->q.peek(st)) {
          const bool bounded = st->get_run_type() == RunType::bounded;
          if (bounded && num_bounded_ >= limit && !pipelines_[i].stage[0].empty()) break;
          queues_[i]->q.pop_always();
          pending_inputs_.fetch_sub(1, std::memory_order_acq_rel);
          if (bounded) ++num_bounded_;
          in_flight_.fetch_add(1, std::memory_order_acq_rel);
          st->start_time = get_time();
          if (trace::enabled()) trace::record_pe_start(st->get_name(), st->get_desc());
          st->start();
          pipelines_[i].stage[0].push_back(st);
        }
      }
    }
    // ---- step ---------------------------------------------------------------
    bool any = false;
    for (size_t i = 0; i < nq; ++i) {
      for (int s = 0; s < AL_PE_NUM_PIPELINE_STAGES; ++s) {
        auto& vec = pipelines_[i].stage[s];
        for (size_t k = 0; k < vec.size();) {
          AlState* st = vec[k];
          any = true;
          if (st->paused_for_advance) { ++k; continue; }
          PEAction a;
          try {
            a = st->step();
          } catch (const std::exception& e) {
            // A state must report failures through its request; one that throws is
            // dropped so that the engine (and every other stream) keeps running.
            std::cerr << "[al] progress engine: " << st->get_name() << " " << st->get_desc() << " threw: " << e.what()
                      << "\n";
            a = PEAction::complete;
          }
          if (a == PEAction::cont) {
            if (hang_s > 0 && !st->hang_reported && get_time() - st->start_time > hang_s) {
              st->hang_reported = true;
              std::function<void(const AlState&, double)> cb;
              { std::lock_guard<std::mutex> g(cb_mu_); cb = hang_cb_; }
              if (cb) cb(*st, get_time() - st->start_time);
              else
                std::cerr << "[al] progress engine: possible hang in " << st->get_name() << " "
                          << st->get_desc() << " after " << (get_time() - st->start_time) << " s\n";
            }
            ++k;
          } else if (a == PEAction::advance) {
            if (s + 1 >= AL_PE_NUM_PIPELINE_STAGES) {
              // No further stage: treat as "keep going" in the last stage.
              ++k;
            } else if (k == 0) {
              vec.erase(vec.begin());
              pipelines_[i].stage[s + 1].push_back(st);
            } else {
              st->paused_for_advance = true;  // must wait for older states of this stage
              ++k;
            }
          } else {  // complete
            vec.erase(vec.begin() + (long)k);
            if (st->get_run_type() == RunType::bounded) --num_bounded_;
            if (trace::enabled()) trace::record_pe_done(st->get_name(), st->get_desc());
            delete st;
            in_flight_.fetch_sub(1, std::memory_order_acq_rel);
          }
        }
        // Release states that were waiting to advance and are now the oldest.
        if (s + 1 < AL_PE_NUM_PIPELINE_STAGES) {
          while (!vec.empty() && vec.front()->paused_for_advance) {
            AlState* st = vec.front();
            st->paused_for_advance = false;
            vec.erase(vec.begin());
            pipelines_[i].stage[s + 1].push_back(st);
          }
        }
      }
    }
    // ---- back-off -------------------------------------------------------------
    if (any || pending_inputs_.load(std::memory_order_acquire) > 0) {
      idle_spins = 0;
    } else {
      ++idle_spins;
      if (idle_spins < 2000) AL_CPU_RELAX();
      else if (idle_spins < 4000) std::this_thread::yield();
      else std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
  }
}

}  // namespace internal
}  // namespace Al
