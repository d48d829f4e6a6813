// How far apart does a host barrier release the ranks?  The timing protocol of the benchmarks (host barrier,
// event, operation, event) charges that distance to the operation.  Measures Al::Barrier<HostBackend> (shared
// memory) and the control plane's socket exchange (Group::barrier); runs on CPU ranks, no GPU needed.
//   alrun -n 8 barrier_skew
#include "Al.hpp"
#include <time.h>
#include <algorithm>
#include <cstdio>
#include <vector>
static double now() { timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec * 1e6 + t.tv_nsec * 1e-3; }
int main(int argc, char** argv) {
  Al::Initialize(argc, argv);
  {
    Al::HostCommunicator comm;
    const int p = comm.size(), r = comm.rank();
    const int iters = 2000;
    for (int mode = 0; mode < 2; ++mode) {
      std::vector<double> t(iters), dur(iters);
      for (int i = 0; i < iters; ++i) {
        const double a = now();
        if (mode == 0) Al::Barrier<Al::HostBackend>(comm); else comm.group().barrier();
        t[i] = now(); dur[i] = t[i] - a;
      }
      std::vector<double> all((size_t)iters * p);
      Al::Gather<Al::HostBackend>(t.data(), all.data(), (size_t)iters, 0, comm);
      if (r == 0) {
        std::vector<double> skew;
        for (int i = 100; i < iters; ++i) { double lo = 1e300, hi = 0; for (int q = 0; q < p; ++q) { lo = std::min(lo, all[(size_t)q * iters + i]); hi = std::max(hi, all[(size_t)q * iters + i]); } skew.push_back(hi - lo); }
        std::sort(skew.begin(), skew.end()); std::sort(dur.begin(), dur.end());
        printf("%s ranks %d: exit skew median %.2f us, p90 %.2f us; barrier time median %.2f us\n", mode == 0 ? "HostCommunicator barrier" : "control-plane barrier", p, skew[skew.size() / 2], skew[skew.size() * 9 / 10], dur[dur.size() / 2]);
      }
    }
  }
  Al::Finalize();
}
