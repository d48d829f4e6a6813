// recover - carrying on after a rank was lost (host backend; works the same way with
// Al::DeviceCommunicator::from_ranks on GPUs).
//
//   alrun -n 4 recover            (also: alrun -n 6 --nodes 2 recover)
//
// The last rank leaves after the first step.  The next collective fails on the others
// (an exception, within milliseconds: the lost rank's control connection is closed);
// they ask which processes are still there, build a communicator over exactly those
// and finish the remaining steps.  The reference has no counterpart: its communicators
// are fixed at creation and a lost rank ends the job.
#include <unistd.h>

#include <algorithm>
#include <cstdio>
#include <vector>

#include "Al.hpp"

int main(int argc, char** argv) {
  Al::Initialize(argc, argv);
  int rc = 0;
  {
    Al::HostCommunicator world;
    const int p = world.size(), me = world.rank();
    std::vector<float> x(1024, 1.f);
    Al::Allreduce<Al::HostBackend>(x.data(), x.size(), Al::ReductionOperator::sum, world);
    if (me == p - 1 && p > 1) {
      printf("rank %d leaves\n", me);
      fflush(stdout);
      _exit(0);  // gone without a word, nothing in flight
    }
    bool failed = p == 1;
    try {
      Al::Allreduce<Al::HostBackend>(x.data(), x.size(), Al::ReductionOperator::sum, world);
    } catch (const Al::al_exception&) {
      failed = true;
    }
    if (!failed) {
      fprintf(stderr, "rank %d: the collective returned although a rank is missing\n", me);
      rc = 2;
    } else {
      std::vector<int> alive = Al::AliveRanks();
      for (int tries = 0; (int)alive.size() != std::max(1, p - 1) && tries < 100; ++tries) alive = Al::AliveRanks();
      Al::HostCommunicator rest = Al::HostCommunicator::from_ranks(alive);
      std::vector<float> y(1024, (float)(rest.rank() + 1));
      for (int step = 0; step < 3; ++step) {
        std::fill(y.begin(), y.end(), (float)(rest.rank() + 1));
        Al::Allreduce<Al::HostBackend>(y.data(), y.size(), Al::ReductionOperator::sum, rest);
      }
      const float want = (float)(rest.size() * (rest.size() + 1) / 2);
      if (y[0] != want || y[1023] != want) rc = 3;
      printf("rank %d: %s with %d of %d ranks\n", me, rc ? "WRONG RESULT" : "carried on", rest.size(), p);
    }
  }
  Al::Finalize();
  return rc;
}
