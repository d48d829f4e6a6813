// API / progress-engine trace logs (see al/trace.hpp).
#include "al/trace.hpp"

#include <unistd.h>

#include <fstream>
#include <mutex>

namespace Al {
namespace trace {

std::atomic<bool> g_enabled{false};

namespace {
std::mutex g_mu;
std::vector<std::string> g_ops, g_pe;
}  // namespace

void enable(bool on) { g_enabled.store(on, std::memory_order_relaxed); }

void append_op(std::string&& line) {
  std::lock_guard<std::mutex> g(g_mu);
  g_ops.emplace_back(std::move(line));
}
void append_pe(std::string&& line) {
  std::lock_guard<std::mutex> g(g_mu);
  g_pe.emplace_back(std::move(line));
}
std::vector<std::string> snapshot() {
  std::lock_guard<std::mutex> g(g_mu);
  std::vector<std::string> out = g_ops;
  out.insert(out.end(), g_pe.begin(), g_pe.end());
  return out;
}
void clear() {
  std::lock_guard<std::mutex> g(g_mu);
  g_ops.clear();
  g_pe.clear();
}
void write(std::ostream& os) {
  std::lock_guard<std::mutex> g(g_mu);
  os << "Trace:\n";
  for (const auto& l : g_ops) os << l << "\n";
  os << "Progress engine trace:\n";
  for (const auto& l : g_pe) os << l << "\n";
}
std::string write_to_file() {
  if (!enabled()) return "";
  char host[256] = "localhost";
  gethostname(host, sizeof(host) - 1);
  std::string dir = internal::env_str("AL_TRACE_DIR", ".");
  std::string path = dir + "/" + host + "." + std::to_string(getpid()) + ".trace.txt";
  std::ofstream f(path);
  if (!f) return "";
  write(f);
  return path;
}
void record_pe_start(const char* name, const std::string& desc) {
  if (!enabled()) return;
  append_pe(build_string(get_time(), " PE START ", name, " ", desc));
}
void record_pe_done(const char* name, const std::string& desc) {
  if (!enabled()) return;
  append_pe(build_string(get_time(), " PE DONE ", name, " ", desc));
}

}  // namespace trace
}  // namespace Al
