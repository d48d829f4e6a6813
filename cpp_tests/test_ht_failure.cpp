// A host exchange that fails must reach the caller of the host-transfer backend: Test / Wait on the
// request and every later call on the communicator throw, and the stream is released instead of
// waiting forever.  The failure is made on the host (the host communicator underneath is aborted
// before the operation); nothing on the GPU faults or hangs.  One process, one GPU.
#include <cstdio>
#include <chrono>
#include <cmath>
#include <thread>
#include <vector>

#include "Al.hpp"
#include "al/cuda/cuda.hpp"

int main() {
  if (!Al::internal::cuda::device_usable()) {
    printf("no CUDA device usable\n");
    return 0;
  }
  int fails = 0;
  auto expect = [&](bool ok, const char* what) {
    if (!ok) { ++fails; fprintf(stderr, "FAILED: %s\n", what); }
  };
  Al::Initialize();
  {
    using B = Al::HostTransferBackend;
    cudaStream_t s;
    AL_CHECK_CUDA(cudaStreamCreate(&s));
    B::comm_type comm(s);
    const size_t n = 1000;
    float* d = nullptr;
    AL_CHECK_CUDA(cudaMalloc(&d, n * sizeof(float)));
    std::vector<float> h(n, 1.5f);
    AL_CHECK_CUDA(cudaMemcpy(d, h.data(), n * sizeof(float), cudaMemcpyHostToDevice));

    // sanity: the healthy path works
    Al::Allreduce<B>(d, n, Al::ReductionOperator::sum, comm);
    AL_CHECK_CUDA(cudaStreamSynchronize(s));
    expect(!comm.failed(), "healthy operation leaves the communicator usable");

    comm.host().abort("injected by the test");
    B::req_type req = B::null_req;
    Al::NonblockingAllreduce<B>(d, n, Al::ReductionOperator::sum, comm, req);
    // The stream must drain although the host exchange never happened.
    cudaError_t e = cudaErrorNotReady;
    for (int i = 0; i < 2000 && e == cudaErrorNotReady; ++i) {
      e = cudaStreamQuery(comm.internal_stream());
      if (e == cudaErrorNotReady) std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    expect(e == cudaSuccess, "the stream is released after the failed exchange");
    bool threw = false;
    try { (void)Al::Test<B>(req); } catch (const Al::al_exception&) { threw = true; }
    expect(threw, "Test rethrows the failure");
    expect(comm.failed(), "the communicator is marked failed");
    threw = false;
    try { Al::Allreduce<B>(d, n, Al::ReductionOperator::sum, comm); } catch (const Al::al_exception&) { threw = true; }
    expect(threw, "later calls on the failed communicator throw");
    AL_CHECK_CUDA(cudaDeviceSynchronize());
    AL_CHECK_CUDA(cudaMemcpy(h.data(), d, n * sizeof(float), cudaMemcpyDeviceToHost));
    expect(std::isnan(h[0]) && std::isnan(h[n - 1]), "the receive buffer of the failed operation is poisoned, not stale");
    AL_CHECK_CUDA(cudaFree(d));
    AL_CHECK_CUDA(cudaStreamDestroy(s));
  }
  Al::Finalize();
  printf(fails ? "ht failure test: FAIL\n" : "ht failure test: ok\n");
  return fails ? 1 : 0;
}
