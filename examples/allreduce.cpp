// allreduce - overlap a non-blocking allreduce with other work and join on the stream.
//   alrun -n 2 allreduce [host|device]
// Shows the semantics this API is built around (examples/allreduce.cpp:46-125 of the reference):
// on a GPU backend "blocking" means stream-ordered, Wait() makes the communicator's stream wait,
// Test() polls from the host, and a Barrier synchronises streams, not hosts.
#include <algorithm>
#include <cstring>
#include <iostream>
#include <vector>

#include "Al.hpp"

template <typename Backend, typename Alloc, typename Free, typename Sync>
void demo(Alloc alloc, Free release, Sync sync) {
  typename Backend::comm_type comm;
  const size_t n = 1 << 20;
  float* buf = alloc(n, (float)(comm.rank() + 1));
  typename Backend::req_type req;
  Al::NonblockingAllreduce<Backend>(buf, n, Al::ReductionOperator::sum, comm, req);
  // ... independent work could be enqueued / executed here ...
  int polls = 0;
  while (!Al::Test<Backend>(req)) ++polls;  // host-side completion check
  Al::Allreduce<Backend>(buf, n, Al::ReductionOperator::max, comm);  // stream-ordered on GPU backends
  Al::Barrier<Backend>(comm);
  const float first = sync(buf, comm);
  const float expect = comm.size() * (comm.size() + 1) / 2.0f;
  std::cout << Backend::Name() << " rank " << comm.rank() << ": value " << first << " (expected " << expect << "), polled "
            << polls << " times" << std::endl;
  release(buf);
}

int main(int argc, char** argv) {
  Al::Initialize(argc, argv);
  if (argc > 1 && !strcmp(argv[1], "device")) {
    demo<Al::DeviceBackend>(
        [](size_t n, float v) { float* d; cudaMalloc((void**)&d, n * 4); std::vector<float> h(n, v); cudaMemcpy(d, h.data(), n * 4, cudaMemcpyHostToDevice); return d; },
        [](float* p) { cudaFree(p); },
        [](float* p, Al::DeviceCommunicator& c) { cudaStreamSynchronize(c.get_stream()); float h; cudaMemcpy(&h, p, 4, cudaMemcpyDeviceToHost); return h; });
  } else {
    demo<Al::HostBackend>([](size_t n, float v) { float* p = new float[n]; std::fill(p, p + n, v); return p; },
                          [](float* p) { delete[] p; }, [](float* p, Al::HostCommunicator&) { return p[0]; });
  }
  Al::Finalize();
  return 0;
}
