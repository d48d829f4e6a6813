// benchmark_ops - times one operation of one backend over a sweep of message sizes.
//
//   alrun -n 8 benchmark_ops --backend device|nccl|host|ht --op allreduce --datatype float
//         [--algo auto|one_shot|two_shot|nvls|ll] [--inplace] [--nonblocking] [--symmetric] [--register] [--check]
//         [--min-bytes 8 --max-bytes 1073741824] [--num-warmup 20] [--num-iters 100]
//         [--reduction-op sum] [--out FILE] [--summarize]
//
// Protocol (that of the reference's benchmark/benchmark_ops.cpp:184-195 and
// benchmark_utils_nccl.hpp:46-58): a host barrier before every iteration, a
// cudaEvent pair on the communicator's stream around the operation (+ Wait for
// non-blocking), event synchronise.  Every iteration's time is reduced with max
// over ranks (a multi-GPU time is the slowest rank's time); rank 0 reports
// median / mean / min / max per size together with the bus bandwidth
// (allreduce S/t*2(p-1)/p, reduce_scatter / allgather / alltoall S/t*(p-1)/p with S the
// full buffer).  `--backend nccl` runs the reference backend's NCCL call sequence.
// --symmetric allocates the buffers with symm_alloc (device) / ncclMemAlloc + ncclCommRegister (nccl);
// --register registers cudaMalloc'ed buffers with Al::RegisterMemory (device backend);
// --check compares the result of every size with the serial oracle on a sample of positions.
//
// Output columns follow the reference's schema (benchmark/benchmark_utils.hpp:155-181)
// with the statistics appended:
//   Backend Type Operation Algo NonBlocking InPlace Root CommSize Bytes Median_us Mean_us Min_us Max_us BusGBs
#include <algorithm>
#include <fstream>
#include <numeric>

#include "../baseline/nccl_equiv.hpp"
#include "../cpp_tests/test_common.hpp"

using namespace altest;
using Al::ReductionOperator;

namespace {

struct Stats { double median, mean, min, max; };
Stats summarize(std::vector<double> v) {
  std::sort(v.begin(), v.end());
  Stats s;
  s.median = v.empty() ? 0 : v[v.size() / 2];
  s.mean = v.empty() ? 0 : std::accumulate(v.begin(), v.end(), 0.0) / (double)v.size();
  s.min = v.empty() ? 0 : v.front();
  s.max = v.empty() ? 0 : v.back();
  return s;
}

double bus_factor(const std::string& op, int p) {
  if (op == "allreduce") return 2.0 * (p - 1) / p;
  if (op == "reduce_scatter" || op == "allgather" || op == "alltoall") return (double)(p - 1) / p;
  return 1.0;
}

struct Timer {
  cudaEvent_t a, b;
  Timer() { cudaEventCreate(&a); cudaEventCreate(&b); }
  ~Timer() { cudaEventDestroy(a); cudaEventDestroy(b); }
};

int nccl_dtype(Al::DType d) {
  switch (d) {
    case Al::DType::f32: return nccl_equiv::Float32;
    case Al::DType::bf16: return nccl_equiv::Bfloat16;
    case Al::DType::f16: return nccl_equiv::Float16;
    case Al::DType::f64: return nccl_equiv::Float64;
    case Al::DType::i32: return nccl_equiv::Int32;
    default: return nccl_equiv::Uint8;
  }
}
int nccl_op(ReductionOperator op) {
  switch (op) {
    case ReductionOperator::prod: return nccl_equiv::Prod;
    case ReductionOperator::min: return nccl_equiv::Min;
    case ReductionOperator::max: return nccl_equiv::Max;
    case ReductionOperator::avg: return nccl_equiv::Avg;
    default: return nccl_equiv::Sum;
  }
}

template <typename T>
void fill_device(T* p, size_t n, int rank) {
  std::minstd_rand rng((unsigned)rank + 1);
  std::vector<T> h(std::min<size_t>(n, 1 << 20));
  for (auto& v : h) v = from_double<T>(((double)(rng() % 20001) - 10000.0) / 10000.0);  // U(-1, 1)
  for (size_t off = 0; off < n; off += h.size())
    cudaMemcpy(p + off, h.data(), std::min(h.size(), n - off) * sizeof(T), cudaMemcpyHostToDevice);
}

/** One benchmark run for element type T on GPU buffers. */
template <typename T>
int run_gpu(const Args& a, const std::string& backend) {
  const ReductionOperator rop = parse_redop(a.str("reduction-op", "sum"));
  const bool inplace = a.has("inplace"), nb = a.has("nonblocking"), symmetric = a.has("symmetric");
  const long warm = a.num("num-warmup", 20), iters = a.num("num-iters", 100);
  const size_t min_b = (size_t)a.num("min-bytes", 8), max_b = (size_t)a.num("max-bytes", 1 << 26);
  auto split_list = [](const std::string& v) {
    std::vector<std::string> out;
    size_t i = 0;
    while (i <= v.size()) {
      size_t j = v.find(',', i);
      if (j == std::string::npos) j = v.size();
      if (j > i) out.push_back(v.substr(i, j - i));
      i = j + 1;
    }
    return out;
  };
  const std::vector<std::string> ops = split_list(a.str("op", "allreduce"));
  const std::vector<std::string> algos = split_list(a.str("algo", "auto"));
  const std::vector<std::string> cta_caps = split_list(a.str("ctas", "0"));

  cudaStream_t stream;
  AL_CHECK_CUDA(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking));
  Al::HostCommunicator hcomm;  // host barrier + max-over-ranks of the timings
  const int p = hcomm.size(), me = hcomm.rank();
  std::unique_ptr<Al::DeviceCommunicator> dcomm;
  std::unique_ptr<Al::HostTransferCommunicator> htcomm;
  std::unique_ptr<nccl_equiv::Communicator> ncomm;
  if (backend == "device") dcomm.reset(new Al::DeviceCommunicator(stream));
  else if (backend == "ht") htcomm.reset(new Al::HostTransferCommunicator(stream));
  else ncomm.reset(new nccl_equiv::Communicator(hcomm.group(), stream));

  // S = bytes of the full buffer (the larger side of the operation)
  const size_t max_elems = std::max<size_t>(1, max_b / sizeof(T));
  T *sbuf = nullptr, *rbuf = nullptr;
  const size_t alloc = (max_elems + (size_t)p) * sizeof(T);
  bool nccl_registered = false;
  if (symmetric && dcomm) {
    sbuf = (T*)dcomm->symm_alloc(alloc);
    rbuf = (T*)dcomm->symm_alloc(alloc);
  } else if (symmetric && ncomm && (sbuf = (T*)ncomm->alloc_registered(alloc)) != nullptr) {
    rbuf = (T*)ncomm->alloc_registered(alloc);
    nccl_registered = true;
  } else {
    AL_CHECK_CUDA(cudaMalloc((void**)&sbuf, alloc));
    AL_CHECK_CUDA(cudaMalloc((void**)&rbuf, alloc));
  }
  fill_device(sbuf, max_elems, me);
  AL_CHECK_CUDA(cudaMemset(rbuf, 0, alloc));
  const bool registered = a.has("register") && dcomm && !symmetric;
  if (registered) {
    Al::RegisterMemory<Al::DeviceBackend>(sbuf, max_elems + (size_t)p, *dcomm);
    Al::RegisterMemory<Al::DeviceBackend>(rbuf, max_elems + (size_t)p, *dcomm);
  }
  // --check: every rank's input block (fill_device repeats one block of at most 1 Mi elements)
  const bool checking = a.has("check") && !inplace;
  const size_t block = std::min<size_t>(max_elems, 1 << 20);
  std::vector<std::vector<double>> blocks;
  if (checking) {
    for (int r = 0; r < p; ++r) {
      std::minstd_rand rng((unsigned)r + 1);
      std::vector<double> b(block);
      for (auto& v : b) v = to_double(from_double<T>(((double)(rng() % 20001) - 10000.0) / 10000.0));
      blocks.push_back(std::move(b));
    }
  }
  long check_failures = 0;

  std::ofstream file;
  if (me == 0 && a.has("out")) file.open(a.str("out", ""), std::ios::app);
  std::ostream& os = file.is_open() ? (std::ostream&)file : (std::ostream&)std::cout;
  if (me == 0 && !a.has("no-header"))
    os << "Backend Type Operation Algo NonBlocking InPlace Root CommSize Bytes Median_us Mean_us Min_us Max_us BusGBs\n";

  Timer tm;
  HangWatchdog dog((double)a.num("hang-timeout", 120));
  const int default_cap = Al::tuning().max_ctas, default_cap_nvls = Al::tuning().max_ctas_nvls, default_cap_zc = Al::tuning().max_ctas_zero_copy;
  for (const std::string& op : ops)
  for (const std::string& algo_name : (op == "allreduce" && dcomm ? algos : std::vector<std::string>{"auto"}))
  for (const std::string& cap_s : cta_caps) {
  const int cap = atoi(cap_s.c_str());
  Al::tuning().max_ctas = cap > 0 ? cap : default_cap;
  Al::tuning().max_ctas_nvls = cap > 0 ? cap : default_cap_nvls;
  Al::tuning().max_ctas_zero_copy = cap > 0 ? cap : default_cap_zc;
  Al::DeviceAllreduceAlgo algo = Al::DeviceAllreduceAlgo::automatic;
  if (algo_name == "one_shot") algo = Al::DeviceAllreduceAlgo::one_shot;
  else if (algo_name == "two_shot") algo = Al::DeviceAllreduceAlgo::two_shot;
  else if (algo_name == "nvls") algo = Al::DeviceAllreduceAlgo::nvls;
  else if (algo_name == "ll") algo = Al::DeviceAllreduceAlgo::ll;
  const std::string algo_s = algo_name + (cap > 0 ? "/c" + cap_s : "");
  if (algo == Al::DeviceAllreduceAlgo::nvls && dcomm && !dcomm->has_multicast()) continue;
  for (size_t bytes = std::max(min_b, sizeof(T)); bytes <= max_b; bytes *= 2) {
    const size_t total = bytes / sizeof(T);                 // elements of the full buffer
    const size_t per = std::max<size_t>(1, total / (size_t)p);  // per-rank slice for the scattered ops
    const bool sliced = op == "reduce_scatter" || op == "allgather" || op == "alltoall";
    if (sliced && total < (size_t)p) continue;
    const T* s = inplace ? (const T*)rbuf : sbuf;
    auto launch = [&](Al::DeviceBackend::req_type& req) {
      if (dcomm) {
        Al::DeviceCommunicator& c = *dcomm;
        if (op == "allreduce") {
          if (nb) inplace ? Al::NonblockingAllreduce<Al::DeviceBackend>(rbuf, total, rop, c, req, algo) : Al::NonblockingAllreduce<Al::DeviceBackend>(s, rbuf, total, rop, c, req, algo);
          else inplace ? Al::Allreduce<Al::DeviceBackend>(rbuf, total, rop, c, algo) : Al::Allreduce<Al::DeviceBackend>(s, rbuf, total, rop, c, algo);
        } else if (op == "reduce_scatter") {
          inplace ? Al::Reduce_scatter<Al::DeviceBackend>(rbuf, per, rop, c) : Al::Reduce_scatter<Al::DeviceBackend>(s, rbuf, per, rop, c);
        } else if (op == "allgather") {
          inplace ? Al::Allgather<Al::DeviceBackend>(rbuf, per, c) : Al::Allgather<Al::DeviceBackend>(s, rbuf, per, c);
        } else if (op == "alltoall") {
          inplace ? Al::Alltoall<Al::DeviceBackend>(rbuf, per, c) : Al::Alltoall<Al::DeviceBackend>(s, rbuf, per, c);
        } else if (op == "bcast") {
          Al::Bcast<Al::DeviceBackend>(rbuf, total, 0, c);
        } else if (op == "reduce") {
          Al::Reduce<Al::DeviceBackend>(s, rbuf, total, rop, 0, c);
        } else if (op == "sendrecv") {
          Al::SendRecv<Al::DeviceBackend>(s, total, (me + 1) % p, rbuf, total, (me + p - 1) % p, c);
        } else if (op == "barrier") {
          Al::Barrier<Al::DeviceBackend>(c);
        } else throw_al_exception("benchmark_ops: unsupported op ", op);
      } else if (htcomm) {
        Al::HostTransferCommunicator& c = *htcomm;
        if (op == "allreduce") Al::Allreduce<Al::HostTransferBackend>(s, rbuf, total, rop, c);
        else if (op == "allgather") Al::Allgather<Al::HostTransferBackend>(s, rbuf, per, c);
        else if (op == "alltoall") Al::Alltoall<Al::HostTransferBackend>(s, rbuf, per, c);
        else if (op == "reduce_scatter") Al::Reduce_scatter<Al::HostTransferBackend>(s, rbuf, per, rop, c);
        else if (op == "bcast") Al::Bcast<Al::HostTransferBackend>(rbuf, total, 0, c);
        else throw_al_exception("benchmark_ops: unsupported op ", op);
      } else {
        nccl_equiv::Communicator& c = *ncomm;
        const int dt = nccl_dtype(Al::TypeMap<T>::value), o = nccl_op(rop);
        if (op == "allreduce") c.allreduce(s, rbuf, total, dt, o);
        else if (op == "reduce_scatter") c.reduce_scatter(s, rbuf, per, dt, o);
        else if (op == "allgather") c.allgather(inplace ? rbuf + (size_t)me * per : s, rbuf, per, dt);
        else if (op == "alltoall") {
          if (inplace) {  // the reference copies the whole buffer to a temporary first (nccl_impl.hpp:1228-1234)
            AL_CHECK_CUDA(cudaMemcpyAsync(sbuf, rbuf, per * (size_t)p * sizeof(T), cudaMemcpyDeviceToDevice, stream));
            c.alltoall(sbuf, rbuf, per, dt, sizeof(T));
          } else c.alltoall(s, rbuf, per, dt, sizeof(T));
        } else if (op == "bcast") c.bcast(rbuf, total, dt, 0);
        else if (op == "reduce") c.reduce(s, rbuf, total, dt, o, 0);
        else if (op == "sendrecv") c.sendrecv(s, total, (me + 1) % p, rbuf, total, (me + p - 1) % p, dt);
        else if (op == "barrier") {  // the reference's barrier is a 1-byte allreduce (nccl_impl.hpp:1080-1090)
          c.allreduce(rbuf, rbuf, 1, nccl_equiv::Uint8, nccl_equiv::Sum);
        } else throw_al_exception("benchmark_ops: unsupported op ", op);
      }
    };
    std::vector<double> times;
    dog.arm(op + " " + std::to_string(bytes) + " bytes");
    for (long it = 0; it < warm + iters; ++it) {
      Al::Barrier<Al::HostBackend>(hcomm);
      Al::DeviceBackend::req_type req = nullptr;
      AL_CHECK_CUDA(cudaEventRecord(tm.a, stream));
      launch(req);
      if (req) Al::Wait<Al::DeviceBackend>(req);
      AL_CHECK_CUDA(cudaEventRecord(tm.b, stream));
      AL_CHECK_CUDA(cudaEventSynchronize(tm.b));
      float ms = 0;
      AL_CHECK_CUDA(cudaEventElapsedTime(&ms, tm.a, tm.b));
      if (it >= warm) times.push_back((double)ms * 1e3);
    }
    dog.disarm();
    if (dcomm) dcomm->check_status();
    if (checking && (op == "allreduce" || sliced)) {
      // expected value of output element i from the ranks' input blocks (input element j of rank r = blocks[r][j % block])
      auto in = [&](int r, size_t j) { return blocks[(size_t)r][j % block]; };
      auto expect = [&](size_t i) -> double {
        if (op == "allgather") return in((int)(i / per), i % per);
        if (op == "alltoall") return in((int)(i / per), (size_t)me * per + i % per);
        const size_t j = op == "allreduce" ? i : (size_t)me * per + i;
        double acc = in(0, j);
        for (int r = 1; r < p; ++r) {
          const double v = in(r, j);
          acc = rop == ReductionOperator::max ? std::max(acc, v) : (rop == ReductionOperator::min ? std::min(acc, v) : acc + v);
        }
        return rop == ReductionOperator::avg ? acc / p : acc;
      };
      const size_t out_n = op == "allreduce" ? total : (op == "reduce_scatter" ? per : per * (size_t)p);
      const size_t head = std::min<size_t>(out_n, 65536), tail = std::min<size_t>(out_n - head, 4096);
      std::vector<T> h(head + tail);
      AL_CHECK_CUDA(cudaMemcpy(h.data(), rbuf, head * sizeof(T), cudaMemcpyDeviceToHost));
      if (tail) AL_CHECK_CUDA(cudaMemcpy(h.data() + head, rbuf + out_n - tail, tail * sizeof(T), cudaMemcpyDeviceToHost));
      const double tol = sizeof(T) == 2 ? 0.05 * p : 1e-4 * p;
      for (size_t k = 0; k < h.size(); ++k) {
        const size_t i = k < head ? k : out_n - tail + (k - head);
        if (std::fabs(to_double(h[k]) - expect(i)) > tol) {
          if (check_failures++ == 0)
            fprintf(stderr, "[rank %d] %s %zu bytes: element %zu is %g, expected %g\n", me, op.c_str(), bytes, i, to_double(h[k]), expect(i));
        }
      }
    }
    // max over ranks, iteration by iteration
    std::vector<double> worst(times.size());
    Al::Allreduce<Al::HostBackend>((const double*)times.data(), worst.data(), times.size(), ReductionOperator::max, hcomm);
    if (me == 0) {
      const Stats st = summarize(worst);
      const double gbs = st.median > 0 ? (double)bytes / (st.median * 1e-6) * bus_factor(op, p) / 1e9 : 0;
      os << backend << ' ' << a.str("datatype", "float") << ' ' << op << ' ' << (dcomm ? algo_s : "-") << ' ' << nb << ' '
         << inplace << " 0 " << p << ' ' << bytes << ' ' << st.median << ' ' << st.mean << ' ' << st.min << ' ' << st.max
         << ' ' << gbs << std::endl;
    }
  }
  }
  AL_CHECK_CUDA(cudaStreamSynchronize(stream));
  Al::Barrier<Al::HostBackend>(hcomm);
  if (registered) {
    Al::UnregisterMemory<Al::DeviceBackend>(sbuf, *dcomm);
    Al::UnregisterMemory<Al::DeviceBackend>(rbuf, *dcomm);
  }
  if (symmetric && dcomm) { dcomm->symm_free(sbuf); dcomm->symm_free(rbuf); }
  else if (nccl_registered) { ncomm->free_registered(sbuf); ncomm->free_registered(rbuf); }
  else { cudaFree(sbuf); cudaFree(rbuf); }
  if (checking) {
    long all_failures = 0;
    std::vector<double> mine{(double)check_failures}, sum(1);
    Al::Allreduce<Al::HostBackend>((const double*)mine.data(), sum.data(), 1, ReductionOperator::sum, hcomm);
    all_failures = (long)sum[0];
    if (me == 0) fprintf(stderr, "benchmark_ops --check: %s\n", all_failures ? "MISMATCHES" : "all sampled results correct");
    check_failures = all_failures;
  }
  dcomm.reset(); htcomm.reset(); ncomm.reset();
  cudaStreamDestroy(stream);
  return check_failures ? 1 : 0;
}

/** Host backend: steady-clock timing (benchmark/benchmark_utils_mpi.hpp:35-45 of the reference). */
template <typename T>
int run_host(const Args& a) {
  const std::string op = a.str("op", "allreduce");
  const ReductionOperator rop = parse_redop(a.str("reduction-op", "sum"));
  const long warm = a.num("num-warmup", 10), iters = a.num("num-iters", 100);
  const size_t min_b = (size_t)a.num("min-bytes", 8), max_b = (size_t)a.num("max-bytes", 1 << 22);
  Al::HostCommunicator comm;
  const int p = comm.size(), me = comm.rank();
  std::vector<T> s(max_b / sizeof(T) + (size_t)p), r(max_b / sizeof(T) + (size_t)p);
  for (size_t i = 0; i < s.size(); ++i) s[i] = from_double<T>((double)((i * 7 + (size_t)me) % 13) / 13.0);
  if (me == 0 && !a.has("no-header"))
    std::cout << "Backend Type Operation Algo NonBlocking InPlace Root CommSize Bytes Median_us Mean_us Min_us Max_us BusGBs\n";
  for (size_t bytes = std::max(min_b, sizeof(T)); bytes <= max_b; bytes *= 2) {
    const size_t total = bytes / sizeof(T), per = std::max<size_t>(1, total / (size_t)p);
    std::vector<double> times;
    for (long it = 0; it < warm + iters; ++it) {
      Al::Barrier<Al::HostBackend>(comm);
      const double t0 = Al::get_time();
      if (op == "allreduce") Al::Allreduce<Al::HostBackend>((const T*)s.data(), r.data(), total, rop, comm);
      else if (op == "allgather") Al::Allgather<Al::HostBackend>((const T*)s.data(), r.data(), per, comm);
      else if (op == "alltoall") Al::Alltoall<Al::HostBackend>((const T*)s.data(), r.data(), per, comm);
      else if (op == "reduce_scatter") Al::Reduce_scatter<Al::HostBackend>((const T*)s.data(), r.data(), per, rop, comm);
      else if (op == "bcast") Al::Bcast<Al::HostBackend>(r.data(), total, 0, comm);
      else throw_al_exception("benchmark_ops: unsupported op ", op);
      if (it >= warm) times.push_back((Al::get_time() - t0) * 1e6);
    }
    std::vector<double> worst(times.size());
    Al::Allreduce<Al::HostBackend>((const double*)times.data(), worst.data(), times.size(), ReductionOperator::max, comm);
    if (me == 0) {
      const Stats st = summarize(worst);
      std::cout << "host " << a.str("datatype", "float") << ' ' << op << " - 0 0 0 " << p << ' ' << bytes << ' ' << st.median
                << ' ' << st.mean << ' ' << st.min << ' ' << st.max << ' '
                << (double)bytes / (st.median * 1e-6) * bus_factor(op, p) / 1e9 << std::endl;
    }
  }
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  Args a(argc, argv);
  try {
    Al::Initialize(argc, argv);
    const std::string b = a.str("backend", "device"), t = a.str("datatype", "float");
    int rc;
    if (b == "host") rc = t == "double" ? run_host<double>(a) : run_host<float>(a);
    else if (t == "float") rc = run_gpu<float>(a, b);
    else if (t == "bfloat16") rc = run_gpu<bf16_t>(a, b);
    else if (t == "half") rc = run_gpu<half_t>(a, b);
    else if (t == "double") rc = run_gpu<double>(a, b);
    else if (t == "int") rc = run_gpu<int>(a, b);
    else throw_al_exception("unsupported datatype ", t);
    Al::Finalize();
    return rc;
  } catch (const std::exception& e) {
    fprintf(stderr, "benchmark_ops: %s\n", e.what());
    return 1;
  }
}
