/**
 * @file progress.hpp
 * The progress engine: one background thread per process that drives every
 * asynchronous host-side state machine (CPU collectives, host-staged GPU
 * transfers, RMA handshakes, watchdogs).
 *
 * Parity: include/aluminum/progress.hpp:64-169 and src/progress.cpp:247-641.
 * Kept semantics:
 *   - one input queue per ordering domain ("stream"), at most AL_PE_NUM_STREAMS;
 *   - per-stream run queues split into AL_PE_NUM_PIPELINE_STAGES stages, a
 *     state may only advance when it is the oldest of its stage;
 *   - bounded states are admitted only while fewer than
 *     `pe_num_concurrent_ops` are running, unless their stream's first stage
 *     is empty; unbounded states are always admitted;
 *   - start on demand; dump_state() for post-mortem; hang watchdog.
 * Differences: input queues are always multi-producer safe; the poll loop
 * backs off (pause -> yield) when nothing is in flight instead of spinning
 * flat out; the thread is bound with sched_setaffinity to the last core of
 * the process' affinity mask minus the local rank (no hwloc dependency).
 */
#pragma once
#include <string>
#include <vector>
#include <atomic>
#include <condition_variable>
#include <functional>
#include <iosfwd>
#include <mutex>
#include <thread>
#include <vector>

#include "al/config.hpp"
#include "al/state.hpp"
#include "al/util/mpsc_queue.hpp"

namespace Al {
namespace internal {

/** "0-3,8,10-11" (the format of sysfs cpulist files) -> the listed core numbers. */
std::vector<int> parse_cpulist(const std::string& text);
/**
 * Core for the progress thread: among the cores the process may use, prefer those local to the GPU
 * (`near_gpu`, may be empty), take the highest-numbered one and step down by the node-local rank.
 * -1 = do not bind (fewer than two cores allowed).
 */
int choose_pe_core(const std::vector<int>& allowed, const std::vector<int>& near_gpu, long local_rank);

class ProgressEngine {
 public:
  ProgressEngine();
  ~ProgressEngine();
  ProgressEngine(const ProgressEngine&) = delete;
  ProgressEngine& operator=(const ProgressEngine&) = delete;

  /** Start the thread (idempotent). */
  void run();
  /** Stop and join; outstanding states are abandoned. */
  void stop();
  bool is_running() const { return started_.load(std::memory_order_acquire); }
  /** Hand a heap-allocated state to the engine, which takes ownership - also when it throws (table or queue full). */
  void enqueue(AlState* state);
  /** Human-readable dump of every run queue. Safe to call from a signal handler context on a best-effort basis. */
  std::ostream& dump_state(std::ostream& os);
  /** Called (from the engine thread) when a state has been stepping longer than the hang threshold. */
  void set_hang_callback(std::function<void(const AlState&, double seconds)> cb);
  /** Device the engine thread makes current before running (set by the CUDA layer). */
  void set_device(int dev) { device_ = dev; }
  /**
   * Tell the engine that an ordering domain is gone (its communicator or
   * stream was destroyed, nothing of it is in flight): the slot can serve a
   * new key.  Without this a process that keeps creating communicators would
   * run out of the AL_PE_NUM_STREAMS slots.
   */
  void release_key(const void* key);
  /** Number of states admitted and not yet completed. */
  size_t in_flight() const { return in_flight_.load(std::memory_order_acquire); }
  /** The core the thread was bound to, or -1. */
  int bound_core() const { return bound_core_; }
  /** How many cores the kernel reported as local to the GPU (0: unknown, the choice fell back to all allowed cores). */
  int near_gpu_cores() const { return near_gpu_cores_; }

 private:
  struct InputQueue {
    explicit InputQueue(const void* k) : key(k), q(AL_PE_INPUT_QUEUE_SIZE) {}
    std::atomic<const void*> key;  ///< read without a lock by enqueue(), changed under add_mu_
    MPSCQueue<AlState*> q;
  };
  struct StreamPipeline {
    std::vector<AlState*> stage[AL_PE_NUM_PIPELINE_STAGES];
  };

  void engine();
  void bind();
  InputQueue* queue_for(const void* key);

  std::thread thread_;
  std::atomic<bool> started_{false};
  std::atomic<bool> stop_flag_{false};
  std::mutex start_mu_;
  bool starting_ = false;  ///< a caller is inside run() creating the thread (guarded by start_mu_)
  std::condition_variable start_cv_;
  bool thread_ready_ = false;

  // Input side: slots are only ever appended (under add_mu_) and published
  // through num_queues_, so the engine thread can scan them without a lock.
  std::mutex add_mu_;
  InputQueue* queues_[AL_PE_NUM_STREAMS] = {};
  std::atomic<size_t> num_queues_{0};

  // Engine-thread private.
  StreamPipeline pipelines_[AL_PE_NUM_STREAMS];
  size_t num_bounded_ = 0;
  std::atomic<size_t> in_flight_{0};
  std::atomic<size_t> pending_inputs_{0};

  std::mutex cb_mu_;
  std::function<void(const AlState&, double)> hang_cb_;
  int device_ = -1;
  int bound_core_ = -1;
  int near_gpu_cores_ = 0;
};

/** The process-wide engine (created by Initialize). */
ProgressEngine* get_progress_engine();
/** The engine, or nullptr when the library is not initialised (destructors that may run after Finalize). */
ProgressEngine* get_progress_engine_if_any();
/** ProgressEngine::release_key on the process's engine, if there is one. */
void release_progress_key(const void* key);

}  // namespace internal
}  // namespace Al
