// bandwidth - uni-directional point-to-point bandwidth between every ordered pair of ranks, one
// pair at a time, printed as a source x destination matrix in GiB/s.
//   alrun -n 8 bandwidth [--backend device|host] [--bytes 268435456] [--iters 10] [--register]
// --register registers the buffers with the communicator first (Al::RegisterMemory): large messages then go
// straight into the receive buffer instead of through the mailbox ring.
// Parity: benchmark/bandwidth.cpp:95-137,193-273 of the reference.
#include "../cpp_tests/test_common.hpp"

using namespace altest;

template <typename Comm> void drain(Comm&) {}
template <> void drain<Al::DeviceCommunicator>(Al::DeviceCommunicator& c) { AL_CHECK_CUDA(cudaStreamSynchronize(c.get_stream())); }

template <typename Backend>
int run(const Args& a) {
  typename Backend::comm_type comm;
  Al::HostCommunicator hc;
  const int p = comm.size(), me = comm.rank();
  const size_t bytes = (size_t)a.num("bytes", 64 << 20), n = bytes / 4;
  const long iters = a.num("iters", 10);
  Buffer<Backend, float> buf(n);
  buf.upload(std::vector<float>(n, (float)me), comm);
  const bool reg = a.has("register");
  if (reg) Al::RegisterMemory<Backend>(buf.data(), n, comm);
  std::vector<double> mat((size_t)(p * p), 0.0);
  for (int s = 0; s < p; ++s)
    for (int d = 0; d < p; ++d) {
      if (s == d) continue;
      Al::Barrier<Al::HostBackend>(hc);
      double dt = 0;
      if (me == s || me == d) {
        for (long it = -2; it < iters; ++it) {
          if (it == 0) drain(comm);
          const double t0 = Al::get_time();
          if (me == s) Al::Send<Backend>((const float*)buf.data(), n, d, comm);
          else Al::Recv<Backend>(buf.data(), n, s, comm);
          if (it == iters - 1) drain(comm);  // the stream must be empty before the clock stops
          if (it >= 0) dt += Al::get_time() - t0;
        }
      }
      if (me == d) mat[(size_t)(s * p + d)] = (double)bytes * (double)iters / dt / (1 << 30);
    }
  std::vector<double> all((size_t)(p * p));
  Al::Allreduce<Al::HostBackend>((const double*)mat.data(), all.data(), mat.size(), Al::ReductionOperator::max, hc);
  if (reg) Al::UnregisterMemory<Backend>(buf.data(), comm);
  if (me == 0) {
    printf("%s send/recv bandwidth%s, %zu bytes, GiB/s (row = source, column = destination)\n", Backend::Name().c_str(),
           reg ? " (registered buffers)" : "", bytes);
    for (int s = 0; s < p; ++s) {
      for (int d = 0; d < p; ++d) printf("%8.1f", all[(size_t)(s * p + d)]);
      printf("\n");
    }
  }
  return 0;
}

int main(int argc, char** argv) {
  Args a(argc, argv);
  try {
    Al::Initialize(argc, argv);
    int rc = a.str("backend", "device") == "host" ? run<Al::HostBackend>(a) : run<Al::DeviceBackend>(a);
    Al::Finalize();
    return rc;
  } catch (const std::exception& e) {
    fprintf(stderr, "bandwidth: %s\n", e.what());
    return 1;
  }
}
