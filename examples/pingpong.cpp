// pingpong - ranks 0 and 1 bounce a message; reports the round-trip time per size.
//   alrun -n 2 pingpong [host|device]
// Parity: examples/pingpong.cpp of the reference.
#include <cstring>
#include <iostream>
#include <vector>

#include "Al.hpp"

template <typename Backend>
void run(float* buf, typename Backend::comm_type& comm, void (*drain)(typename Backend::comm_type&)) {
  if (comm.size() < 2) { std::cout << "pingpong needs two ranks" << std::endl; return; }
  for (size_t n = 1; n <= (1 << 20); n *= 16) {
    const int iters = 200;
    drain(comm);
    const double t0 = Al::get_time();
    for (int i = 0; i < iters; ++i) {
      if (comm.rank() == 0) { Al::Send<Backend>((const float*)buf, n, 1, comm); Al::Recv<Backend>(buf, n, 1, comm); }
      else if (comm.rank() == 1) { Al::Recv<Backend>(buf, n, 0, comm); Al::Send<Backend>((const float*)buf, n, 0, comm); }
    }
    drain(comm);
    if (comm.rank() == 0)
      std::cout << Backend::Name() << " " << n * 4 << " bytes: " << (Al::get_time() - t0) / iters * 1e6 << " us per round trip" << std::endl;
  }
}

int main(int argc, char** argv) {
  Al::Initialize(argc, argv);
  if (argc > 1 && !strcmp(argv[1], "device")) {
    Al::DeviceCommunicator comm;
    float* d;
    cudaMalloc((void**)&d, (1 << 20) * 4);
    cudaMemset(d, 0, (1 << 20) * 4);
    run<Al::DeviceBackend>(d, comm, [](Al::DeviceCommunicator& c) { cudaStreamSynchronize(c.get_stream()); });
    cudaFree(d);
  } else {
    Al::HostCommunicator comm;
    std::vector<float> h(1 << 20, 1.f);
    run<Al::HostBackend>(h.data(), comm, [](Al::HostCommunicator&) {});
  }
  Al::Finalize();
  return 0;
}
