// test_rma - the one-sided extension on device communicators.
//   alrun -n 4 test_rma --mode ring|halo [--max-size 1048576]
// ring: every rank attaches the buffers of both ring neighbours, puts a vector to the right
//       neighbour, notifies it, waits for the left neighbour's notify and checks what arrived; then
//       the same in the other direction (test/test_rma_ring.cpp:38-108 of the reference).
// halo: ranks form a 2-D grid (rows x cols), every rank puts one vector to each of its up to four
//       neighbours between two Syncs (test/test_rma_halo_exchange.cpp:79-241).
// Attach is pairwise collective: pairs are visited in an order both sides agree on (lower peer
// first; even ranks attach right-then-left, odd ranks left-then-right on the ring).
#include <algorithm>

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
  // Both neighbours at once (all notifies, then all waits): one Sync per neighbour in ring order would make
  // every rank wait for its right neighbour before it signals its left one - a cycle from four ranks on.
  const int both[2] = {right, left};
  Al::ext::Sync(both, left != right ? 2 : 1, comm);
  Al::ext::DetachRemoteBuffer(r_right, right, comm);
  Al::ext::DetachRemoteBuffer(r_left, left, comm);
  // The buffers are released on return: every importer must have closed its mapping first.
  Al::Barrier<Al::DeviceBackend>(comm);
  AL_CHECK_CUDA(cudaStreamSynchronize(comm.get_stream()));
  return ok;
}

// 2-D halo exchange on a rows x cols grid without wrap-around.  Direction d of a rank: 0 up,
// 1 down, 2 left, 3 right; d ^ 1 is the direction in which the neighbour sees this rank.
// Every rank owns, per direction, a source vector, a landing buffer and an echo buffer.
//   attach   landing and echo buffers, pair by pair;
//   Sync;    put source d into the neighbour's landing buffer;            Sync; check landing
//   put      what landed from d back into that neighbour's echo buffer;   Sync; check echo == source
//   Sync;    detach.
// Boundary ranks pass the null peer (-1), for which every call is a no-op.
static bool halo(Al::DeviceCommunicator& comm, size_t n, int rows, int cols) {
  const int me = comm.rank();
  const int r = me / cols, c = me % cols;
  int nb[4] = {r > 0 ? me - cols : -1, r + 1 < rows ? me + cols : -1, c > 0 ? me - 1 : -1, c + 1 < cols ? me + 1 : -1};
  cudaStream_t s = comm.get_stream();
  std::vector<DeviceBuf<float>> src, land, echo;
  std::vector<std::vector<float>> src_h;
  for (int d = 0; d < 4; ++d) {
    src.emplace_back(n + 1); land.emplace_back(n + 1); echo.emplace_back(n + 1);
    src_h.push_back(gen_data<float>(n + 1, me, Al::ReductionOperator::sum, (unsigned)d + 1));
    src[(size_t)d].upload_on(src_h.back(), s);
    land[(size_t)d].upload_on(std::vector<float>(n + 1, -1.f), s);
    echo[(size_t)d].upload_on(std::vector<float>(n + 1, -2.f), s);
  }
  // Attach is pairwise collective.  Every rank visits its neighbours in ascending rank order: a
  // cycle of ranks each waiting for a neighbour that is busy with a lower-numbered one cannot close.
  int order[4] = {0, 1, 2, 3};
  std::sort(order, order + 4, [&](int a, int b) { return nb[a] < nb[b]; });
  float* r_land[4] = {nullptr, nullptr, nullptr, nullptr};
  float* r_echo[4] = {nullptr, nullptr, nullptr, nullptr};
  for (int k = 0; k < 4; ++k) {
    const int d = order[k];
    r_land[d] = Al::ext::AttachRemoteBuffer(land[(size_t)d].data(), nb[d], comm);  // the neighbour's landing buffer for what comes from me
    r_echo[d] = Al::ext::AttachRemoteBuffer(echo[(size_t)d].data(), nb[d], comm);
  }
  Al::ext::Sync(nb, 4, comm);
  for (int d = 0; d < 4; ++d) Al::ext::Put(src[(size_t)d].data(), nb[d], r_land[d], n, comm);
  Al::ext::Sync(nb, 4, comm);
  bool ok = true;
  for (int d = 0; d < 4; ++d) {
    if (nb[d] < 0) continue;
    auto want = gen_data<float>(n + 1, nb[d], Al::ReductionOperator::sum, (unsigned)(d ^ 1) + 1);
    auto got = land[(size_t)d].download_on(s);
    ok = ok && got[n] == -1.f;  // nothing written past the end
    want.resize(n); got.resize(n);
    ok = check_vector(got, want, "halo landing", me) && ok;
  }
  for (int d = 0; d < 4; ++d) Al::ext::Put(land[(size_t)d].data(), nb[d], r_echo[d], n, comm);
  Al::ext::Sync(nb, 4, comm);
  for (int d = 0; d < 4; ++d) {
    if (nb[d] < 0) continue;
    auto want = src_h[(size_t)d];
    auto got = echo[(size_t)d].download_on(s);
    ok = ok && got[n] == -2.f;
    want.resize(n); got.resize(n);
    ok = check_vector(got, want, "halo echo", me) && ok;
  }
  Al::ext::Sync(nb, 4, comm);  // nobody is still writing into a buffer that is about to be released
  for (int k = 0; k < 4; ++k) {
    const int d = order[k];
    Al::ext::DetachRemoteBuffer(r_echo[d], nb[d], comm);
    Al::ext::DetachRemoteBuffer(r_land[d], nb[d], comm);
  }
  // The buffers are released on return: every importer must have closed its mapping first.
  Al::Barrier<Al::DeviceBackend>(comm);
  AL_CHECK_CUDA(cudaStreamSynchronize(s));
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
      if (a.str("mode", "ring") == "halo") {
        const int p = comm.size();
        int rows = 1;
        for (int q = 1; q * q <= p; ++q)
          if (p % q == 0) rows = q;
        rows = (int)a.num("rows", rows);
        if (rows < 1 || p % rows != 0) throw_al_exception("--rows must divide the number of ranks");
        for (size_t n : sweep_sizes(1, (size_t)a.num("max-size", 1 << 20), true, true)) {
          dog.arm("rma halo " + std::to_string(n));
          if (!halo(comm, n, rows, p / rows)) { ++failed; break; }
          dog.disarm();
        }
        comm.check_status();
        if (comm.rank() == 0)
          printf("DeviceBackend rma halo grid=%dx%d: %s\n", rows, p / rows, failed ? "FAIL" : "ok");
      }
      for (size_t n : sweep_sizes(1, (size_t)a.num("max-size", 1 << 20), true, true)) {
        if (a.str("mode", "ring") != "ring") break;
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
      if (comm.rank() == 0 && a.str("mode", "ring") == "ring")
        printf("DeviceBackend rma ring ranks=%d: %s\n", comm.size(), failed ? "FAIL" : "ok");
    }
    Al::Finalize();
    return failed ? 1 : 0;
  } catch (const std::exception& e) {
    fprintf(stderr, "test_rma: %s\n", e.what());
    return 1;
  }
}
