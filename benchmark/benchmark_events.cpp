// benchmark_events - cost of learning on the host that a stream reached a point: the pinned-flag
// "event" (GPUStatusFlag: cuStreamWriteValue32 + host load) against cudaEventRecord / cudaEventQuery,
// measured as host time to record and time until the host observes completion behind a short
// delay kernel.  Parity: benchmark/benchmark_events.cpp:76-109, benchmark/wait.cu:38-46.
#include <cstdio>

#include "Al.hpp"
#include "al/cuda/gpu_status_flag.hpp"
#include "al/cuda/helper_kernels.hpp"

using namespace Al::internal::cuda;

int main(int argc, char** argv) {
  const int iters = argc > 1 ? atoi(argv[1]) : 2000;
  Al::Initialize();
  if (!device_usable()) { printf("no CUDA device\n"); return 0; }
  cudaStream_t s;
  AL_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
  cudaEvent_t ev;
  AL_CHECK_CUDA(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
  double rec_flag = 0, obs_flag = 0, rec_ev = 0, obs_ev = 0;
  GPUStatusFlag flag;
  for (int i = 0; i < iters; ++i) {
    launch_delay_kernel(s, 20000);
    double t0 = Al::get_time();
    flag.record(s);
    rec_flag += Al::get_time() - t0;
    t0 = Al::get_time();
    while (!flag.query()) {}
    obs_flag += Al::get_time() - t0;
    launch_delay_kernel(s, 20000);
    t0 = Al::get_time();
    AL_CHECK_CUDA(cudaEventRecord(ev, s));
    rec_ev += Al::get_time() - t0;
    t0 = Al::get_time();
    while (cudaEventQuery(ev) == cudaErrorNotReady) {}
    obs_ev += Al::get_time() - t0;
  }
  printf("pinned flag   record %.2f us   observe (incl. 20 us delay kernel) %.2f us\n", rec_flag / iters * 1e6, obs_flag / iters * 1e6);
  printf("cuda event    record %.2f us   observe (incl. 20 us delay kernel) %.2f us\n", rec_ev / iters * 1e6, obs_ev / iters * 1e6);
  AL_CHECK_CUDA(cudaEventDestroy(ev));
  AL_CHECK_CUDA(cudaStreamDestroy(s));
  Al::Finalize();
  return 0;
}
