// test_rma - the one-sided extension on device communicators.
//   alrun -n 4 test_rma --mode ring|halo [--max-size 1048576]
// ring: every rank attaches the buffers of both ring neighbours, puts a vector to the right
//       neighbour, notifies it, waits for the left neighbour's notify and checks what arrived; then
//       the same in the other direction (test/test_rma_ring.cpp:38-108 of the reference).
// halo: ranks form a 2-D grid (rows x cols), every rank puts one vector to each of its up to four
//       neighbours between two Syncs (test/test_rma_halo_exchange.cpp:79-241).
// Attach is pairwise collective: pairs are visited in an order both sides agree on (lower peer
// first; even ranks attach right-then-left, odd ranks left-then-right on the ring).
#include "test_common.hpp"

using namespace altest;

static bool ring(Al::DeviceCommunicator& comm, size_t n) {
  const int p = comm.size(), me = comm.rank();
  const int right = (me + 1) % p, left = (me + p - 1) % p;
  DeviceBuf<float> from_left(n + 1), from_right(n + 1), src(n + 1);
  src.upload_on(gen_data<float>(n + 1, me, Al::ReductionOperator::sum), comm.get_stream());
  float *r_right = nullptr, *r_left = nullptr;  // neighbours' landing buffers as mapped here
  // An attach is a pairwise exchange: I hand over the buffer the peer may write into and receive the
  // one it handed over in its matching call.  Towards the right neighbour I offer my "from_right"
  // buffer and obtain its "from_left" buffer, and vice versa.
  auto attach_right = [&] { r_right = Al::ext::AttachRemoteBuffer(from_right.data(), right, comm); };
  auto attach_left = [&] { r_left = Al::ext::AttachRemoteBuffer(from_left.data(), left, comm); };
  if (me % 2 == 0) { attach_right(); attach_left(); }
  else { attach_left(); attach_right(); }
  Al::ext::Put(src.data(), right, r_right, n, comm);   // lands in right's from_left
  Al::ext::Notify(right, comm);
  Al::ext::Wait(left, comm);
  Al::ext::Put(src.data(), left, r_left, n, comm);     // lands in left's from_right
  Al::ext::Notify(left, comm);
  Al::ext::Wait(right, comm);
  auto want_l = gen_data<float>(n + 1, left, Al::ReductionOperator::sum);
  auto want_r = gen_data<float>(n + 1, right, Al::ReductionOperator::sum);
  want_l.resize(n); want_r.resize(n);
  auto got_l = from_left.download_on(comm.get_stream());
  auto got_r = from_right.download_on(comm.get_stream());
  got_l.resize(n); got_r.resize(n);
  const bool ok = check_vector(got_l, want_l, "ring from left", me) && check_vector(got_r, want_r, "ring from right", me);
  Al::ext::Sync(right, comm);
  if (left != right) Al::ext::Sync(left, comm);
  Al::ext::DetachRemoteBuffer(r_right, right, comm);
  Al::ext::DetachRemoteBuffer(r_left, left, comm);
  return ok;
}

int main(int argc, char** argv) {
  Args a(argc, argv);
  try {
    Al::Initialize(argc, argv);
    int failed = 0;
    {
      Al::DeviceCommunicator comm;
      HangWatchdog dog(60);
      for (size_t n : sweep_sizes(1, (size_t)a.num("max-size", 1 << 20), true, true)) {
        dog.arm("rma ring " + std::to_string(n));
        if (!ring(comm, n)) { ++failed; break; }
        dog.disarm();
      }
      // null and self connections
      float* none = Al::ext::AttachRemoteBuffer((float*)nullptr, -1, comm);
      Al::ext::Notify(-1, comm);
      Al::ext::Wait(-1, comm);
      Al::ext::Sync(-1, comm);
      DeviceBuf<float> self(16);
      float* me_ptr = Al::ext::AttachRemoteBuffer(self.data(), comm.rank(), comm);
      if (none != nullptr || me_ptr != self.data()) ++failed;
      comm.check_status();
      if (comm.rank() == 0) printf("DeviceBackend rma ring ranks=%d: %s\n", comm.size(), failed ? "FAIL" : "ok");
    }
    Al::Finalize();
    return failed ? 1 : 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "test_rma: %s\n", e.what());
    return 1;
  }
}
