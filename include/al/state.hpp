/**
 * @file state.hpp
 * The unit of work of the progress engine: a small state machine that is
 * started once and then stepped until it reports completion.
 *
 * Parity: include/aluminum/state.hpp:38-108 (AlState, PEAction, RunType).
 */
#pragma once
#include <atomic>
#include <memory>
#include <string>

#include "al/profiling.hpp"

namespace Al {

/** Host-side completion flag shared between an operation and its request. */
using HostRequest = std::shared_ptr<std::atomic<bool>>;
inline HostRequest make_host_request() { return std::make_shared<std::atomic<bool>>(false); }

namespace internal {

/** What the engine should do with a state after a step. */
enum class PEAction {
  cont,      ///< keep stepping in the current pipeline stage
  advance,   ///< move to the next pipeline stage (in issue order per stream)
  complete   ///< finished: remove and destroy
};

/** Bounded states count against the engine's concurrency limit; unbounded ones
 *  (point-to-point, which may wait arbitrarily long for a partner) do not. */
enum class RunType { bounded, unbounded };

class AlState {
 public:
  AlState() = default;
  virtual ~AlState() { profiling::prof_end(range_); }
  AlState(const AlState&) = delete;
  AlState& operator=(const AlState&) = delete;

  /** Called once by the engine when the state is admitted. */
  virtual void start() { range_ = profiling::prof_start(get_name()); }
  /** Called repeatedly; must not block. */
  virtual PEAction step() = 0;
  /**
   * Ordering domain.  States with the same key are admitted in enqueue order
   * and advance through pipeline stages in that order.  Device-related states
   * return the CUDA stream they were enqueued on; host states return their
   * communicator.
   */
  virtual const void* get_compute_stream() const { return nullptr; }
  virtual RunType get_run_type() const { return RunType::bounded; }
  virtual const char* get_name() const { return "AlState"; }
  virtual std::string get_desc() const { return ""; }

  // engine bookkeeping
  bool paused_for_advance = false;
  double start_time = 0.0;
  bool hang_reported = false;

 private:
  profiling::ProfileRange range_;
};

}  // namespace internal
}  // namespace Al
