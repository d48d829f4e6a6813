/**
 * @file trace.hpp
 * In-memory API trace: one line per library call plus progress-engine
 * start/done records, written to "<host>.<pid>.trace.txt" at Finalize() or
 * from the fatal-signal handler.
 *
 * Parity: include/aluminum/trace.hpp:67-104, src/trace.cpp:54-114.  The
 * reference compiles the recorder out unless AL_TRACE is configured; here it
 * is always compiled and gated by one relaxed atomic load (AL_TRACE=1 or
 * Al::trace::enable()).
 */
#pragma once
#include <atomic>
#include <sstream>
#include <string>
#include <vector>

#include "al/base.hpp"
#include "al/util/utils.hpp"

namespace Al {
namespace trace {

extern std::atomic<bool> g_enabled;
inline bool enabled() { return g_enabled.load(std::memory_order_relaxed); }
void enable(bool on);

/** Append one already-formatted line to the API log. */
void append_op(std::string&& line);
/** Append one line to the progress-engine log. */
void append_pe(std::string&& line);
/** Copy of both logs (API first), for tests. */
std::vector<std::string> snapshot();
void clear();
/** Write both logs to `os`. */
void write(std::ostream& os);
/** Write to "<hostname>.<pid>.trace.txt" in AL_TRACE_DIR (default "."); returns the path or "". */
std::string write_to_file();

namespace detail {
inline void put(std::ostringstream&) {}
template <typename A, typename... R>
void put(std::ostringstream& ss, const A& a, const R&... r) {
  ss << ' ' << a;
  put(ss, r...);
}
template <typename A>
void put_ptr(std::ostringstream& ss, const A* p) { ss << ' ' << static_cast<const void*>(p); }
}  // namespace detail

/**
 * Record "time backend dtype op rank size args...".
 * Pointers print as addresses, vectors as their length.
 */
template <typename... Args>
void record_op(const char* backend, DType dt, const char* op, int rank, int size, const Args&... args) {
  if (!enabled()) return;
  std::ostringstream ss;
  ss.precision(9);
  ss << std::fixed << get_time() << ' ' << backend << ' ' << dtype_name(dt) << ' ' << op << ' '
     << rank << ' ' << size;
  detail::put(ss, args...);
  append_op(ss.str());
}

void record_pe_start(const char* name, const std::string& desc);
void record_pe_done(const char* name, const std::string& desc);

}  // namespace trace
}  // namespace Al
