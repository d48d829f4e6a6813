// test_exchange - halo-style neighbour exchange: every rank posts non-blocking SendRecvs with its
// +-k neighbours, waits for all of them, and checks what arrived.
//   alrun -n 4 test_exchange [--backend host|device] [--peers 2] [--size 1024]
// Parity: test/test_exchange.cpp:36-106 (whose main never dispatches to the test body; this one does).
#include "test_common.hpp"

using namespace altest;

template <typename Backend>
int run(const Args& a) {
  typename Backend::comm_type comm;
  const int p = comm.size(), me = comm.rank();
  const int k = (int)std::min<long>(a.num("peers", 2), std::max(1, (p - 1) / 2));
  const size_t n = (size_t)a.num("size", 1024);
  if (p < 2) return 0;
  std::vector<Buffer<Backend, float>> sb, rb;
  std::vector<typename Backend::req_type> reqs((size_t)(2 * k));
  sb.reserve((size_t)(2 * k)); rb.reserve((size_t)(2 * k));
  std::vector<int> dests, srcs;
  for (int d = 1; d <= k; ++d) { dests.push_back((me + d) % p); srcs.push_back((me - d + p) % p); }
  for (int d = 1; d <= k; ++d) { dests.push_back((me - d + p) % p); srcs.push_back((me + d) % p); }
  for (size_t i = 0; i < dests.size(); ++i) {
    sb.emplace_back(n);
    rb.emplace_back(n);
    sb.back().upload(gen_data<float>(n, me, Al::ReductionOperator::sum, (unsigned)dests[i] + 1), comm);
    rb.back().upload(std::vector<float>(n, 0.f), comm);
  }
  for (size_t i = 0; i < dests.size(); ++i)
    Al::NonblockingSendRecv<Backend>((const float*)sb[i].data(), n, dests[i], rb[i].data(), n, srcs[i], comm, reqs[i]);
  for (auto& r : reqs) Al::Wait<Backend>(r);
  bool ok = true;
  for (size_t i = 0; i < srcs.size(); ++i)
    ok = check_vector(rb[i].download(comm), gen_data<float>(n, srcs[i], Al::ReductionOperator::sum, (unsigned)me + 1), "exchange", me) && ok;
  if (me == 0) printf("%s exchange peers=%d size=%zu ranks=%d: %s\n", Backend::Name().c_str(), k, n, p, ok ? "ok" : "FAIL");
  return ok ? 0 : 1;
}

int main(int argc, char** argv) {
  Args a(argc, argv);
  try {
    Al::Initialize(argc, argv);
    int rc = a.str("backend", "host") == "device" ? run<Al::DeviceBackend>(a) : run<Al::HostBackend>(a);
    Al::Finalize();
    return rc;
  } catch (const std::exception& e) {
    fprintf(stderr, "test_exchange: %s\n", e.what());
    return 1;
  }
}
