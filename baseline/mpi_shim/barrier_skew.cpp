// Exit skew of MPI_Barrier(MPI_COMM_WORLD) of the single-node MPI stand-in (shared memory; MPISHIM_NO_SHM=1
// selects the message schedule instead).  Ranks are plain processes:
//   g++ -O2 -std=c++17 -Ibaseline/_ref/mpi/include baseline/mpi_shim/barrier_skew.cpp -Lbaseline/_ref/mpi/lib -lmpi \
//       -Wl,-rpath,$PWD/baseline/_ref/mpi/lib -o barrier_skew_mpi
//   for r in 0 1 2 3; do MPISHIM_JOB=skew MPISHIM_SIZE=4 MPISHIM_RANK=$r ./barrier_skew_mpi & done; wait
#include <mpi.h>
#include <time.h>
#include <algorithm>
#include <cstdio>
#include <vector>
static double now() { timespec t; clock_gettime(CLOCK_MONOTONIC, &t); return t.tv_sec * 1e6 + t.tv_nsec * 1e-3; }
int main(int argc, char** argv) {
  MPI_Init(&argc, &argv);
  int r, p; MPI_Comm_rank(MPI_COMM_WORLD, &r); MPI_Comm_size(MPI_COMM_WORLD, &p);
  const int iters = 2000;
  std::vector<double> t(iters), dur(iters);
  for (int i = 0; i < iters; ++i) { const double a = now(); MPI_Barrier(MPI_COMM_WORLD); t[i] = now(); dur[i] = t[i] - a; }
  std::vector<double> all((size_t)iters * p);
  MPI_Gather(t.data(), iters, MPI_DOUBLE, all.data(), iters, MPI_DOUBLE, 0, MPI_COMM_WORLD);
  if (r == 0) {
    std::vector<double> skew;
    for (int i = 100; i < iters; ++i) { double lo = 1e300, hi = 0; for (int q = 0; q < p; ++q) { lo = std::min(lo, all[(size_t)q * iters + i]); hi = std::max(hi, all[(size_t)q * iters + i]); } skew.push_back(hi - lo); }
    std::sort(skew.begin(), skew.end()); std::sort(dur.begin(), dur.end());
    printf("ranks %d: exit skew median %.2f us, p90 %.2f us; barrier time median %.2f us\n", p, skew[skew.size() / 2], skew[skew.size() * 9 / 10], dur[dur.size() / 2]);
  }
  MPI_Finalize();
}
