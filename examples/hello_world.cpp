// hello_world - every rank contributes its rank number; after an allreduce all ranks print the sum.
//   alrun -n 4 hello_world            (CPU ranks)
//   alrun -n 4 hello_world device     (one GPU per rank)
// Parity: examples/hello_world.cpp of the reference.
#include <cstring>
#include <iostream>

#include "Al.hpp"

int main(int argc, char** argv) {
  Al::Initialize(argc, argv);
  const bool device = argc > 1 && !strcmp(argv[1], "device");
  if (device) {
    Al::DeviceCommunicator comm;
    float h = (float)comm.rank(), *d = nullptr;
    AL_CHECK_CUDA(cudaMalloc((void**)&d, sizeof(float)));
    AL_CHECK_CUDA(cudaMemcpy(d, &h, sizeof(float), cudaMemcpyHostToDevice));
    Al::Allreduce<Al::DeviceBackend>(d, 1, Al::ReductionOperator::sum, comm);  // stream-ordered: returns at once
    AL_CHECK_CUDA(cudaStreamSynchronize(comm.get_stream()));
    AL_CHECK_CUDA(cudaMemcpy(&h, d, sizeof(float), cudaMemcpyDeviceToHost));
    std::cout << "rank " << comm.rank() << " of " << comm.size() << " (device): sum of ranks = " << h << std::endl;
    cudaFree(d);
  } else {
    Al::HostCommunicator comm;
    float v = (float)comm.rank();
    Al::Allreduce<Al::HostBackend>(&v, 1, Al::ReductionOperator::sum, comm);
    std::cout << "rank " << comm.rank() << " of " << comm.size() << " (host): sum of ranks = " << v << std::endl;
  }
  Al::Finalize();
  return 0;
}
