// stress_progress - many small non-blocking allreduces in flight at once.
//
//   alrun -n 8 stress_progress [--ops 64] [--streams 8] [--rounds 20] [--min-bytes 4096] [--max-bytes 262144]
//                              [--backend device|host]
//
// Per rank: `streams` CUDA streams, one device communicator per stream (the library's
// model: a communicator is bound to a stream), `ops` NonblockingAllreduce calls with
// log-uniform fp32 sizes (seed 1, identical on every rank) spread round-robin over the
// communicators, each followed by Wait.  With AL_REQ_MEMOPS=1 both the completion record
// and the Wait are stream memory operations (cuStreamWriteValue32 / cuStreamWaitValue32),
// so nothing in the loop synchronises with the host.  Reports operations per second
// (max over ranks of the round time) and the p50 / p99 of the per-operation device time.
// --backend host runs the same pattern on host memory: `streams` host communicators, all
// operations started before the first Wait, so the progress thread has `ops` states queued
// at once (it admits a bounded number per communicator); times are host clock.
#include <algorithm>
#include <random>

#include "../cpp_tests/test_common.hpp"

using namespace altest;

// The host form of the stress: every operation of a round is started before any is waited for.
static int stress_host(const Args& a) {
  const int nops = (int)a.num("ops", 64), ncomms = (int)a.num("streams", 8), rounds = (int)a.num("rounds", 20);
  const double lo = std::log((double)a.num("min-bytes", 4096)), hi = std::log((double)a.num("max-bytes", 262144));
  Al::HostCommunicator hc;
  std::vector<Al::HostCommunicator> comms;
  for (int i = 0; i < ncomms; ++i) comms.push_back(hc.copy());
  std::mt19937 rng(1);
  std::uniform_real_distribution<double> U(lo, hi);
  std::vector<std::vector<float>> bufs((size_t)nops);
  for (auto& b : bufs) b.assign(std::max<size_t>(1, (size_t)std::exp(U(rng)) / 4), 1.0f);
  std::vector<double> round_us, op_us;
  std::vector<Al::HostBackend::req_type> reqs((size_t)nops);
  std::vector<double> t_start((size_t)nops);
  for (int r = 0; r < rounds + 3; ++r) {
    Al::Barrier<Al::HostBackend>(hc);
    const double t0 = Al::get_time();
    for (int i = 0; i < nops; ++i) {
      t_start[(size_t)i] = Al::get_time();
      Al::NonblockingAllreduce<Al::HostBackend>(bufs[(size_t)i].data(), bufs[(size_t)i].size(), Al::ReductionOperator::max,
                                                comms[(size_t)(i % ncomms)], reqs[(size_t)i]);
    }
    for (int i = 0; i < nops; ++i) {
      Al::Wait<Al::HostBackend>(reqs[(size_t)i]);
      if (r >= 3) op_us.push_back((Al::get_time() - t_start[(size_t)i]) * 1e6);
    }
    if (r >= 3) round_us.push_back((Al::get_time() - t0) * 1e6);
  }
  for (auto& b : bufs)
    if (b.front() != 1.0f || b.back() != 1.0f) throw_al_exception("wrong result");
  std::vector<double> worst(round_us.size());
  Al::Allreduce<Al::HostBackend>((const double*)round_us.data(), worst.data(), round_us.size(), Al::ReductionOperator::max, hc);
  std::sort(worst.begin(), worst.end());
  std::sort(op_us.begin(), op_us.end());
  if (hc.rank() == 0) {
    const double med = worst[worst.size() / 2];
    printf("stress backend=host ranks=%d communicators=%d ops=%d round_median_us=%.1f ops_per_s=%.0f op_p50_us=%.1f op_p99_us=%.1f\n",
           hc.size(), ncomms, nops, med, nops / (med * 1e-6), op_us[op_us.size() / 2], op_us[(size_t)(op_us.size() * 0.99)]);
  }
  Al::Barrier<Al::HostBackend>(hc);
  return 0;
}

int main(int argc, char** argv) {
  Args a(argc, argv);
  try {
    // Non-blocking operations run on pooled internal streams; with the default pool of one stream they would
    // queue behind each other on the device.  One internal stream per compute stream unless the caller chose.
    setenv("AL_CUDA_STREAM_POOL_SIZE", std::to_string(a.num("streams", 8)).c_str(), 0);
    Al::Initialize(argc, argv);
    if (a.str("backend", "device") == "host") {
      const int rc = stress_host(a);
      Al::Finalize();
      return rc;
    }
    const int nops = (int)a.num("ops", 64), nstreams = (int)a.num("streams", 8), rounds = (int)a.num("rounds", 20);
    const double lo = std::log((double)a.num("min-bytes", 4096)), hi = std::log((double)a.num("max-bytes", 262144));
    Al::HostCommunicator hc;
    // One communicator per operation (--comms, default = --ops) spread over the streams: operations of one
    // communicator are chained by design, so only operations of different communicators are truly concurrent.
    // The messages are small: give every communicator a small workspace.
    const int ncomms = (int)a.num("comms", nops);
    Al::tuning().dev_stage_bytes = std::max<size_t>((size_t)a.num("max-bytes", 262144) * 8, size_t{1} << 20);
    Al::tuning().dev_mailbox_bytes = 65536;
    std::vector<cudaStream_t> streams((size_t)nstreams);
    std::vector<std::unique_ptr<Al::DeviceCommunicator>> comms;
    for (auto& s : streams) AL_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    for (int i = 0; i < ncomms; ++i) comms.emplace_back(new Al::DeviceCommunicator(streams[(size_t)(i % nstreams)]));
    std::mt19937 rng(1);
    std::uniform_real_distribution<double> U(lo, hi);
    std::vector<size_t> counts((size_t)nops);
    std::vector<float*> bufs((size_t)nops);
    for (int i = 0; i < nops; ++i) {
      counts[(size_t)i] = std::max<size_t>(1, (size_t)std::exp(U(rng)) / 4);
      AL_CHECK_CUDA(cudaMalloc((void**)&bufs[(size_t)i], counts[(size_t)i] * 4));
      std::vector<float> h(counts[(size_t)i], 1.0f);
      AL_CHECK_CUDA(cudaMemcpy(bufs[(size_t)i], h.data(), h.size() * 4, cudaMemcpyHostToDevice));
    }
    std::vector<cudaEvent_t> e0((size_t)nops), e1((size_t)nops);
    for (int i = 0; i < nops; ++i) { cudaEventCreate(&e0[(size_t)i]); cudaEventCreate(&e1[(size_t)i]); }
    std::vector<double> round_us, op_us;
    for (int r = 0; r < rounds + 3; ++r) {
      Al::Barrier<Al::HostBackend>(hc);
      const double t0 = Al::get_time();
      // every operation is issued before the first Wait: all of them are outstanding at once
      std::vector<Al::DeviceBackend::req_type> reqs((size_t)nops);
      for (int i = 0; i < nops; ++i) {
        Al::DeviceCommunicator& c = *comms[(size_t)(i % ncomms)];
        AL_CHECK_CUDA(cudaEventRecord(e0[(size_t)i], c.get_stream()));
        Al::NonblockingAllreduce<Al::DeviceBackend>(bufs[(size_t)i], counts[(size_t)i], Al::ReductionOperator::max, c, reqs[(size_t)i]);
      }
      for (int i = 0; i < nops; ++i) {
        Al::DeviceCommunicator& c = *comms[(size_t)(i % ncomms)];
        Al::Wait<Al::DeviceBackend>(reqs[(size_t)i]);  // stream-side join, the host continues
        AL_CHECK_CUDA(cudaEventRecord(e1[(size_t)i], c.get_stream()));
      }
      for (auto s : streams) AL_CHECK_CUDA(cudaStreamSynchronize(s));
      const double dt = (Al::get_time() - t0) * 1e6;
      if (r >= 3) {
        round_us.push_back(dt);
        for (int i = 0; i < nops; ++i) {
          float ms = 0;
          cudaEventElapsedTime(&ms, e0[(size_t)i], e1[(size_t)i]);
          op_us.push_back(ms * 1e3);
        }
      }
    }
    for (auto& c : comms) c->check_status();
    // correctness: max of ones is one
    std::vector<float> h(counts[0]);
    AL_CHECK_CUDA(cudaMemcpy(h.data(), bufs[0], counts[0] * 4, cudaMemcpyDeviceToHost));
    if (h[0] != 1.0f || h.back() != 1.0f) throw_al_exception("wrong result");
    std::vector<double> worst(round_us.size());
    Al::Allreduce<Al::HostBackend>((const double*)round_us.data(), worst.data(), round_us.size(), Al::ReductionOperator::max, hc);
    std::sort(worst.begin(), worst.end());
    std::sort(op_us.begin(), op_us.end());
    if (hc.rank() == 0) {
      const double med = worst[worst.size() / 2];
      printf("stress ranks=%d streams=%d comms=%d ops=%d memops=%s round_median_us=%.1f ops_per_s=%.0f op_p50_us=%.1f op_p99_us=%.1f\n",
             hc.size(), nstreams, ncomms, nops, getenv("AL_REQ_MEMOPS") ? getenv("AL_REQ_MEMOPS") : "0", med, nops / (med * 1e-6),
             op_us[op_us.size() / 2], op_us[(size_t)(op_us.size() * 0.99)]);
    }
    Al::Barrier<Al::HostBackend>(hc);
    comms.clear();
    Al::Finalize();
  } catch (const std::exception& e) {
    fprintf(stderr, "stress_progress: %s\n", e.what());
    return 1;
  }
  return 0;
}
