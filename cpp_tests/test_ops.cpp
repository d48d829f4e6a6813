// test_ops - runs any operation of any backend over a sweep of sizes and checks
// every rank's result against a serial oracle computed in the test process.
//
//   alrun -n 4 test_ops --backend host|device|ht --op allreduce --datatype float [--register]
//         [--inplace] [--nonblocking] [--reduction-op sum] [--root 0]
//         [--size N | --min-size A --max-size B] [--odd-sizes] [--zero] [--trials K]
//         [--threads N] [--permute 2,0,1,...]
//
// Parity: test/test_ops.cpp (driver), test/op_runner.hpp (per-op buffer
// conventions).  The reference's oracle is MPI itself; here every rank can
// regenerate every other rank's input, so the expected output is computed
// locally and no second communication library is needed.
#include "test_common.hpp"

using namespace altest;
using Al::ReductionOperator;

namespace {

struct Case {
  std::string op;
  size_t n;
  bool inplace, nonblocking;
  ReductionOperator redop;
  int root;
  bool reg = false;  ///< --register: Al::RegisterMemory on the buffers of the collectives (test/test_ops.cpp:364-367,494 of the reference)
};

/**
 * --register: registers a test buffer with the communicator for the life of the guard.  Registration is
 * collective on the device backend (every rank registers its buffer of the same role, in the same order);
 * the host backends ignore it.  A rank whose buffer is empty (rooted operations) still takes part.
 */
template <typename Backend, typename T>
struct RegGuard {
  typename Backend::comm_type& comm;
  T* ptr = nullptr;
  bool on;
  RegGuard(bool enable, Buffer<Backend, T>& b, typename Backend::comm_type& c) : comm(c), ptr(b.data()), on(enable) {
    if (on) Al::RegisterMemory<Backend>(ptr, b.size(), comm);
  }
  ~RegGuard() {
    if (on) Al::UnregisterMemory<Backend>(ptr, comm);
  }
};

template <typename Backend>
void finish(typename Backend::req_type& req, bool nonblocking) {
  if (nonblocking) Al::Wait<Backend>(req);
}

template <typename T>
std::vector<T> cat(const std::vector<std::vector<T>>& parts) {
  std::vector<T> out;
  for (auto& p : parts) out.insert(out.end(), p.begin(), p.end());
  return out;
}

template <typename Backend, typename T>
bool run_case(const Case& c, typename Backend::comm_type& comm) {
  const int p = comm.size(), me = comm.rank();
  const size_t n = c.n;
  typename Backend::req_type req = Backend::null_req;
  const bool nb = c.nonblocking, ip = c.inplace;
  const ReductionOperator rop = c.redop;
  auto input_of = [&](int r, size_t len, unsigned tag = 0) { return gen_data<T>(len, r, rop, tag); };
  const T fill = from_double<T>(0);

  if (c.op == "allreduce" || c.op == "reduce") {
    std::vector<std::vector<T>> ins;
    for (int r = 0; r < p; ++r) ins.push_back(input_of(r, n));
    std::vector<T> want = reduce_oracle(ins, rop);
    Buffer<Backend, T> in(n), out(n);
    RegGuard<Backend, T> reg_in(c.reg, in, comm), reg_out(c.reg, out, comm);
    in.upload(ins[(size_t)me], comm);
    out.upload(std::vector<T>(n, fill), comm);
    const bool is_ar = c.op == "allreduce";
    if (is_ar) {
      if (ip && nb) Al::NonblockingAllreduce<Backend>(in.data(), n, rop, comm, req);
      else if (ip) Al::Allreduce<Backend>(in.data(), n, rop, comm);
      else if (nb) Al::NonblockingAllreduce<Backend>((const T*)in.data(), out.data(), n, rop, comm, req);
      else Al::Allreduce<Backend>((const T*)in.data(), out.data(), n, rop, comm);
    } else {
      if (ip && nb) Al::NonblockingReduce<Backend>(in.data(), n, rop, c.root, comm, req);
      else if (ip) Al::Reduce<Backend>(in.data(), n, rop, c.root, comm);
      else if (nb) Al::NonblockingReduce<Backend>((const T*)in.data(), out.data(), n, rop, c.root, comm, req);
      else Al::Reduce<Backend>((const T*)in.data(), out.data(), n, rop, c.root, comm);
    }
    finish<Backend>(req, nb);
    bool ok = true;
    if (is_ar || me == c.root) ok = check_vector((ip ? in : out).download(comm), want, c.op.c_str(), me);
    if (!ip) ok = check_vector(in.download(comm), ins[(size_t)me], "input untouched", me) && ok;
    return ok;
  }

  if (c.op == "reduce_scatter" || c.op == "reduce_scatterv") {
    const bool v = c.op == "reduce_scatterv";
    std::vector<size_t> counts((size_t)p);
    for (int r = 0; r < p; ++r) counts[(size_t)r] = v ? n + (size_t)r : n;
    const std::vector<size_t> displs = Al::excl_prefix_sum(counts);
    const size_t total = displs.back() + counts.back();
    std::vector<std::vector<T>> ins;
    for (int r = 0; r < p; ++r) ins.push_back(input_of(r, total));
    std::vector<std::vector<T>> mine;
    for (int r = 0; r < p; ++r)
      mine.emplace_back(ins[(size_t)r].begin() + (long)displs[(size_t)me], ins[(size_t)r].begin() + (long)(displs[(size_t)me] + counts[(size_t)me]));
    std::vector<T> want = reduce_oracle(mine, rop);
    Buffer<Backend, T> in(total), out(counts[(size_t)me]);
    RegGuard<Backend, T> reg_in(c.reg, in, comm), reg_out(c.reg, out, comm);
    in.upload(ins[(size_t)me], comm);
    out.upload(std::vector<T>(counts[(size_t)me], fill), comm);
    if (!v) {
      if (ip && nb) Al::NonblockingReduce_scatter<Backend>(in.data(), n, rop, comm, req);
      else if (ip) Al::Reduce_scatter<Backend>(in.data(), n, rop, comm);
      else if (nb) Al::NonblockingReduce_scatter<Backend>((const T*)in.data(), out.data(), n, rop, comm, req);
      else Al::Reduce_scatter<Backend>((const T*)in.data(), out.data(), n, rop, comm);
    } else {
      if (ip && nb) Al::NonblockingReduce_scatterv<Backend>(in.data(), counts, rop, comm, req);
      else if (ip) Al::Reduce_scatterv<Backend>(in.data(), counts, rop, comm);
      else if (nb) Al::NonblockingReduce_scatterv<Backend>((const T*)in.data(), out.data(), counts, rop, comm, req);
      else Al::Reduce_scatterv<Backend>((const T*)in.data(), out.data(), counts, rop, comm);
    }
    finish<Backend>(req, nb);
    std::vector<T> got = (ip ? in : out).download(comm);
    got.resize(counts[(size_t)me]);
    return check_vector(got, want, c.op.c_str(), me);
  }

  if (c.op == "allgather" || c.op == "allgatherv" || c.op == "gather" || c.op == "gatherv") {
    const bool v = c.op.back() == 'v';
    const bool rooted = c.op[0] == 'g';
    std::vector<size_t> counts((size_t)p);
    for (int r = 0; r < p; ++r) counts[(size_t)r] = v ? n + (size_t)(r % 3) : n;
    const std::vector<size_t> displs = Al::excl_prefix_sum(counts);
    const size_t total = displs.back() + counts.back();
    std::vector<std::vector<T>> ins;
    for (int r = 0; r < p; ++r) ins.push_back(input_of(r, counts[(size_t)r]));
    std::vector<T> want = cat(ins);
    const bool big_in_place = ip && (!rooted || me == c.root);
    Buffer<Backend, T> in(ip ? (big_in_place ? total : counts[(size_t)me]) : counts[(size_t)me]);
    Buffer<Backend, T> out(ip ? 0 : total);
    if (big_in_place) {
      std::vector<T> init(total, fill);
      std::copy(ins[(size_t)me].begin(), ins[(size_t)me].end(), init.begin() + (long)displs[(size_t)me]);
      in.upload(init, comm);
    } else {
      in.upload(ins[(size_t)me], comm);
    }
    if (!ip) out.upload(std::vector<T>(total, fill), comm);
    if (c.op == "allgather") {
      if (ip && nb) Al::NonblockingAllgather<Backend>(in.data(), n, comm, req);
      else if (ip) Al::Allgather<Backend>(in.data(), n, comm);
      else if (nb) Al::NonblockingAllgather<Backend>((const T*)in.data(), out.data(), n, comm, req);
      else Al::Allgather<Backend>((const T*)in.data(), out.data(), n, comm);
    } else if (c.op == "allgatherv") {
      if (ip && nb) Al::NonblockingAllgatherv<Backend>(in.data(), counts, displs, comm, req);
      else if (ip) Al::Allgatherv<Backend>(in.data(), counts, displs, comm);
      else if (nb) Al::NonblockingAllgatherv<Backend>((const T*)in.data(), out.data(), counts, displs, comm, req);
      else Al::Allgatherv<Backend>((const T*)in.data(), out.data(), counts, displs, comm);
    } else if (c.op == "gather") {
      if (ip && nb) Al::NonblockingGather<Backend>(in.data(), n, c.root, comm, req);
      else if (ip) Al::Gather<Backend>(in.data(), n, c.root, comm);
      else if (nb) Al::NonblockingGather<Backend>((const T*)in.data(), out.data(), n, c.root, comm, req);
      else Al::Gather<Backend>((const T*)in.data(), out.data(), n, c.root, comm);
    } else {
      if (ip && nb) Al::NonblockingGatherv<Backend>(in.data(), counts, displs, c.root, comm, req);
      else if (ip) Al::Gatherv<Backend>(in.data(), counts, displs, c.root, comm);
      else if (nb) Al::NonblockingGatherv<Backend>((const T*)in.data(), out.data(), counts, displs, c.root, comm, req);
      else Al::Gatherv<Backend>((const T*)in.data(), out.data(), counts, displs, c.root, comm);
    }
    finish<Backend>(req, nb);
    if (rooted && me != c.root) return check_vector(in.download(comm), ins[(size_t)me], "non-root input untouched", me);
    return check_vector((ip ? in : out).download(comm), want, c.op.c_str(), me);
  }

  if (c.op == "scatter" || c.op == "scatterv") {
    const bool v = c.op == "scatterv";
    std::vector<size_t> counts((size_t)p);
    for (int r = 0; r < p; ++r) counts[(size_t)r] = v ? n + (size_t)(r % 3) : n;
    const std::vector<size_t> displs = Al::excl_prefix_sum(counts);
    const size_t total = displs.back() + counts.back();
    std::vector<T> root_data = input_of(c.root, total);
    std::vector<T> want(root_data.begin() + (long)displs[(size_t)me], root_data.begin() + (long)(displs[(size_t)me] + counts[(size_t)me]));
    const bool root = me == c.root;
    Buffer<Backend, T> in(root ? total : (ip ? counts[(size_t)me] : 0)), out(ip ? 0 : counts[(size_t)me]);
    RegGuard<Backend, T> reg_in(c.reg, in, comm), reg_out(c.reg, out, comm);
    if (root) in.upload(root_data, comm);
    else if (ip) in.upload(std::vector<T>(counts[(size_t)me], fill), comm);
    if (!ip) out.upload(std::vector<T>(counts[(size_t)me], fill), comm);
    if (!v) {
      if (ip && nb) Al::NonblockingScatter<Backend>(in.data(), n, c.root, comm, req);
      else if (ip) Al::Scatter<Backend>(in.data(), n, c.root, comm);
      else if (nb) Al::NonblockingScatter<Backend>((const T*)in.data(), out.data(), n, c.root, comm, req);
      else Al::Scatter<Backend>((const T*)in.data(), out.data(), n, c.root, comm);
    } else {
      if (ip && nb) Al::NonblockingScatterv<Backend>(in.data(), counts, displs, c.root, comm, req);
      else if (ip) Al::Scatterv<Backend>(in.data(), counts, displs, c.root, comm);
      else if (nb) Al::NonblockingScatterv<Backend>((const T*)in.data(), out.data(), counts, displs, c.root, comm, req);
      else Al::Scatterv<Backend>((const T*)in.data(), out.data(), counts, displs, c.root, comm);
    }
    finish<Backend>(req, nb);
    if (ip && root) return check_vector(in.download(comm), root_data, "root buffer unchanged", me);
    return check_vector((ip ? in : out).download(comm), want, c.op.c_str(), me);
  }

  if (c.op == "alltoall" || c.op == "alltoallv") {
    const bool v = c.op == "alltoallv";
    auto cnt = [&](int a, int b) { return v ? n + (size_t)((a + b) % 3) : n; };  // symmetric in (a, b)
    std::vector<size_t> counts((size_t)p);
    for (int r = 0; r < p; ++r) counts[(size_t)r] = cnt(me, r);
    const std::vector<size_t> displs = Al::excl_prefix_sum(counts);
    const size_t total = displs.back() + counts.back();
    std::vector<T> mine = input_of(me, total);
    std::vector<T> want(total);
    for (int r = 0; r < p; ++r) {
      // what rank r sends to me: slice `me` of its send buffer
      std::vector<size_t> rc((size_t)p);
      for (int d = 0; d < p; ++d) rc[(size_t)d] = cnt(r, d);
      const std::vector<size_t> rd = Al::excl_prefix_sum(rc);
      std::vector<T> theirs = input_of(r, rd.back() + rc.back());
      std::copy(theirs.begin() + (long)rd[(size_t)me], theirs.begin() + (long)(rd[(size_t)me] + rc[(size_t)me]),
                want.begin() + (long)displs[(size_t)r]);
    }
    Buffer<Backend, T> in(total), out(ip ? 0 : total);
    RegGuard<Backend, T> reg_in(c.reg, in, comm), reg_out(c.reg, out, comm);
    in.upload(mine, comm);
    if (!ip) out.upload(std::vector<T>(total, fill), comm);
    if (!v) {
      if (ip && nb) Al::NonblockingAlltoall<Backend>(in.data(), n, comm, req);
      else if (ip) Al::Alltoall<Backend>(in.data(), n, comm);
      else if (nb) Al::NonblockingAlltoall<Backend>((const T*)in.data(), out.data(), n, comm, req);
      else Al::Alltoall<Backend>((const T*)in.data(), out.data(), n, comm);
    } else {
      if (ip && nb) Al::NonblockingAlltoallv<Backend>(in.data(), counts, displs, comm, req);
      else if (ip) Al::Alltoallv<Backend>(in.data(), counts, displs, comm);
      else if (nb) Al::NonblockingAlltoallv<Backend>((const T*)in.data(), counts, displs, out.data(), counts, displs, comm, req);
      else Al::Alltoallv<Backend>((const T*)in.data(), counts, displs, out.data(), counts, displs, comm);
    }
    finish<Backend>(req, nb);
    return check_vector((ip ? in : out).download(comm), want, c.op.c_str(), me);
  }

  if (c.op == "bcast") {
    std::vector<T> want = input_of(c.root, n);
    Buffer<Backend, T> buf(n);
    RegGuard<Backend, T> reg_buf(c.reg, buf, comm);
    buf.upload(me == c.root ? want : std::vector<T>(n, fill), comm);
    if (nb) Al::NonblockingBcast<Backend>(buf.data(), n, c.root, comm, req);
    else Al::Bcast<Backend>(buf.data(), n, c.root, comm);
    finish<Backend>(req, nb);
    return check_vector(buf.download(comm), want, "bcast", me);
  }

  if (c.op == "barrier") {
    if (nb) Al::NonblockingBarrier<Backend>(comm, req);
    else Al::Barrier<Backend>(comm);
    finish<Backend>(req, nb);
    Buffer<Backend, T> dummy(1);
    (void)dummy.download(comm);  // synchronises the stream on GPU backends
    return true;
  }

  if (c.op == "send" || c.op == "recv" || c.op == "pt2pt") {
    // even ranks send to rank+1, odd ranks receive; an unpaired last rank idles
    const int partner = (me % 2 == 0) ? me + 1 : me - 1;
    if (partner >= p) return true;
    Buffer<Backend, T> buf(n);
    if (me % 2 == 0) {
      buf.upload(input_of(me, n), comm);
      if (nb) Al::NonblockingSend<Backend>((const T*)buf.data(), n, partner, comm, req);
      else Al::Send<Backend>((const T*)buf.data(), n, partner, comm);
      finish<Backend>(req, nb);
      return check_vector(buf.download(comm), input_of(me, n), "send buffer untouched", me);
    }
    buf.upload(std::vector<T>(n, fill), comm);
    if (nb) Al::NonblockingRecv<Backend>(buf.data(), n, partner, comm, req);
    else Al::Recv<Backend>(buf.data(), n, partner, comm);
    finish<Backend>(req, nb);
    return check_vector(buf.download(comm), input_of(partner, n), "recv", me);
  }

  if (c.op == "sendrecv") {
    const int dest = (me + 1) % p, src = (me - 1 + p) % p;
    Buffer<Backend, T> in(n), out(ip ? 0 : n);
    RegGuard<Backend, T> reg_in(c.reg, in, comm), reg_out(c.reg, out, comm);
    in.upload(input_of(me, n), comm);
    if (!ip) out.upload(std::vector<T>(n, fill), comm);
    if (ip && nb) Al::NonblockingSendRecv<Backend>(in.data(), n, dest, src, comm, req);
    else if (ip) Al::SendRecv<Backend>(in.data(), n, dest, src, comm);
    else if (nb) Al::NonblockingSendRecv<Backend>((const T*)in.data(), n, dest, out.data(), n, src, comm, req);
    else Al::SendRecv<Backend>((const T*)in.data(), n, dest, out.data(), n, src, comm);
    finish<Backend>(req, nb);
    return check_vector((ip ? in : out).download(comm), input_of(src, n), "sendrecv", me);
  }

  if (c.op == "multisendrecv") {
    // every rank exchanges a distinct vector with every other rank
    std::vector<Buffer<Backend, T>> sb, rb;
    std::vector<int> peers;
    for (int r = 0; r < p; ++r) if (r != me) peers.push_back(r);
    sb.reserve(peers.size());
    rb.reserve(peers.size());
    for (int r : peers) {
      sb.emplace_back(n);
      sb.back().upload(input_of(me, n, (unsigned)r + 1), comm);
      if (!ip) { rb.emplace_back(n); rb.back().upload(std::vector<T>(n, fill), comm); }
    }
    std::vector<size_t> counts(peers.size(), n);
    if (ip) {
      std::vector<T*> bufs;
      for (auto& b : sb) bufs.push_back(b.data());
      if (nb) Al::NonblockingMultiSendRecv<Backend>(bufs, counts, peers, peers, comm, req);
      else Al::MultiSendRecv<Backend>(bufs, counts, peers, peers, comm);
    } else {
      std::vector<const T*> sp;
      std::vector<T*> rp;
      for (auto& b : sb) sp.push_back(b.data());
      for (auto& b : rb) rp.push_back(b.data());
      if (nb) Al::NonblockingMultiSendRecv<Backend>(sp, counts, peers, rp, counts, peers, comm, req);
      else Al::MultiSendRecv<Backend>(sp, counts, peers, rp, counts, peers, comm);
    }
    finish<Backend>(req, nb);
    bool ok = true;
    for (size_t k = 0; k < peers.size(); ++k)
      ok = check_vector((ip ? sb[k] : rb[k]).download(comm), input_of(peers[k], n, (unsigned)me + 1), "multisendrecv", me) && ok;
    return ok;
  }
  throw_al_exception("unknown op ", c.op);
}

/** A communicator for one test thread: same ranks, its own stream where the backend has streams. */
template <typename Backend>
typename Backend::comm_type make_thread_comm(const typename Backend::comm_type& comm) {
  if constexpr (std::is_same<typename Backend::comm_type, Al::HostCommunicator>::value) {
    return comm.copy();
  } else {
#ifdef AL_HAS_CUDA
    cudaStream_t s = nullptr;
    AL_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    return comm.copy(s);
#else
    return comm.copy();
#endif
  }
}

template <typename Backend>
void release_thread_comm(typename Backend::comm_type& comm) {
  if constexpr (!std::is_same<typename Backend::comm_type, Al::HostCommunicator>::value) {
#ifdef AL_HAS_CUDA
    cudaStream_t s = comm.get_stream();
    AL_CHECK_CUDA(cudaStreamSynchronize(s));
    { typename Backend::comm_type dying = std::move(comm); }
    AL_CHECK_CUDA(cudaStreamDestroy(s));
#endif
  }
}

/** Runs every size of the sweep on one communicator; returns the number of failed sizes (stops at the first). */
template <typename Backend, typename T>
int sweep(typename Backend::comm_type& comm, Case c, const std::vector<size_t>& sizes, long trials, HangWatchdog& dog) {
  for (size_t n : sizes) {
    for (long t = 0; t < trials; ++t) {
      c.n = n;
      dog.arm(c.op + " size " + std::to_string(n));
      bool ok = false;
      try {
        ok = run_case<Backend, T>(c, comm);
      } catch (const std::exception& e) {
        fprintf(stderr, "[rank %d] %s size %zu threw: %s\n", comm.rank(), c.op.c_str(), n, e.what());
      }
      dog.disarm();
      if (!ok) return 1;
    }
  }
  return 0;
}

/** "--permute 2,0,1": rank i of the world becomes rank list[i] of the tested communicator. */
inline std::vector<int> parse_permutation(const std::string& s, int size) {
  std::vector<int> perm;
  size_t pos = 0;
  while (pos <= s.size()) {
    const size_t comma = s.find(',', pos);
    const std::string tok = s.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos);
    if (!tok.empty()) perm.push_back(std::stoi(tok));
    if (comma == std::string::npos) break;
    pos = comma + 1;
  }
  if ((int)perm.size() != size) throw_al_exception("--permute wants ", size, " entries, got ", perm.size());
  std::vector<int> seen((size_t)size, 0);
  for (int v : perm) {
    if (v < 0 || v >= size || seen[(size_t)v]++) throw_al_exception("--permute is not a permutation of 0..", size - 1);
  }
  return perm;
}

template <typename Backend, typename T>
int run_all(const Args& a) {
  typename Backend::comm_type world;
  // Tested communicator: the world, or the world with its ranks permuted
  // (test/test_utils.hpp:308-334 of the reference does the same with MPI_Comm_split).
  typename Backend::comm_type comm = a.has("permute")
      ? world.split(1, parse_permutation(a.str("permute", ""), world.size())[(size_t)world.rank()])
      : world.copy();
  HangWatchdog dog((double)a.num("hang-timeout", 60));
  Case c;
  c.op = a.str("op", "allreduce");
  c.inplace = a.has("inplace");
  c.nonblocking = a.has("nonblocking");
  c.redop = parse_redop(a.str("reduction-op", "sum"));
  c.root = (int)a.num("root", 0) % comm.size();
  c.reg = a.has("register");
  std::vector<size_t> sizes;
  if (a.has("size")) sizes.push_back((size_t)a.num("size", 1));
  else sizes = sweep_sizes((size_t)a.num("min-size", 1), (size_t)a.num("max-size", 1 << 16), a.has("odd-sizes"), a.has("zero"));
  const long trials = a.num("trials", 1);
  if (c.op == "comm") {  // communicator life cycle only
    for (long t = 0; t < trials; ++t) { typename Backend::comm_type extra = comm.copy(); (void)extra; }
    return 0;
  }
  const int nthreads = (int)a.num("threads", 1);
  int failed = 0;
  if (nthreads <= 1) {
    failed = sweep<Backend, T>(comm, c, sizes, trials, dog);
  } else {
    // Thread-multiple: one communicator per thread (created here, in the same
    // order on every rank), all threads inside the library at once.  Two
    // threads never share a communicator (test/test_ops.cpp:373-391 of the reference).
    std::vector<typename Backend::comm_type> comms;
    for (int t = 0; t < nthreads; ++t) comms.push_back(make_thread_comm<Backend>(comm));
    int thread_device = -1;
#ifdef AL_HAS_CUDA
    if (Al::internal::cuda::device_usable()) (void)cudaGetDevice(&thread_device);
#endif
    std::vector<int> rc((size_t)nthreads, 0);
    std::vector<std::thread> th;
    for (int t = 0; t < nthreads; ++t)
      th.emplace_back([&, t] {
#ifdef AL_HAS_CUDA
        if (thread_device >= 0) (void)cudaSetDevice(thread_device);  // the test's own copies need it; the library sets it itself
#endif
        rc[(size_t)t] = sweep<Backend, T>(comms[(size_t)t], c, sizes, trials, dog);
      });
    for (auto& x : th) x.join();
    for (int r : rc) failed += r;
    for (auto& cm : comms) release_thread_comm<Backend>(cm);
  }
  if (comm.rank() == 0 && !a.has("quiet"))
    printf("%s %s %s%s%s%s sizes=%zu ranks=%d%s: %s\n", Backend::Name().c_str(), c.op.c_str(),
           a.str("datatype", "float").c_str(), c.inplace ? " inplace" : "", c.nonblocking ? " nonblocking" : "",
           a.has("permute") ? " permuted" : "", sizes.size(), comm.size(),
           nthreads > 1 ? (" threads=" + std::to_string(nthreads)).c_str() : "", failed ? "FAIL" : "ok");
  return failed;
}

template <typename Backend>
int by_type(const Args& a) {
  const std::string t = a.str("datatype", "float");
  if (t == "float") return run_all<Backend, float>(a);
  if (t == "double") return run_all<Backend, double>(a);
  if (t == "int") return run_all<Backend, int>(a);
  if (t == "uint") return run_all<Backend, unsigned>(a);
  if (t == "char") return run_all<Backend, signed char>(a);
  if (t == "uchar") return run_all<Backend, unsigned char>(a);
  if (t == "short") return run_all<Backend, short>(a);
  if (t == "llong") return run_all<Backend, long long>(a);
  if (t == "ullong") return run_all<Backend, unsigned long long>(a);
  if (t == "half") return run_all<Backend, half_t>(a);
  if (t == "bfloat16") return run_all<Backend, bf16_t>(a);
  throw_al_exception("unknown datatype ", t);
}

}  // namespace

int main(int argc, char** argv) {
  Args a(argc, argv);
  int rc = 1;
  try {
    Al::Initialize(argc, argv);
    const std::string b = a.str("backend", "host");
    if (b == "host" || b == "mpi") rc = by_type<Al::HostBackend>(a);
#ifdef AL_HAS_CUDA
    else if (b == "device" || b == "nccl") rc = by_type<Al::DeviceBackend>(a);
    else if (b == "ht") rc = by_type<Al::HostTransferBackend>(a);
#endif
    else throw_al_exception("unknown backend ", b);
    Al::Finalize();
  } catch (const std::exception& e) {
    fprintf(stderr, "test_ops: %s\n", e.what());
    return 1;
  }
  return rc ? 1 : 0;
}
