// Check of the MPI stand-in: the unmodified reference library (built without CUDA) runs its MPI
// backend on top of it, and every result is compared with a value computed locally.  One process
// per rank; ranks come from RANK / WORLD_SIZE.  Exit code 0 = every check passed on this rank.
#include <Al.hpp>

#include <cmath>
#include <cstdio>
#include <vector>

namespace {
int g_fail = 0;
int g_rank = 0;
void expect(bool ok, const char* what) {
  if (!ok) { ++g_fail; fprintf(stderr, "[rank %d] FAILED: %s\n", g_rank, what); }
}
float val(int rank, size_t i) { return (float)((rank + 1) * 0.5 + (double)(i % 97) * 0.25); }
}  // namespace

int main(int argc, char** argv) {
  Al::Initialize(argc, argv);
  {
    using B = Al::MPIBackend;
    B::comm_type comm;
    const int p = comm.size(), me = comm.rank();
    g_rank = me;
    expect(comm.local_size() == p, "local communicator covers the node");
    const size_t n = 100003;

    // blocking in-place allreduce
    std::vector<float> a(n);
    for (size_t i = 0; i < n; ++i) a[i] = val(me, i);
    Al::Allreduce<B>(a.data(), n, Al::ReductionOperator::sum, comm);
    bool ok = true;
    for (size_t i = 0; i < n; ++i) {
      float want = 0;
      for (int r = 0; r < p; ++r) want += val(r, i);
      ok = ok && std::fabs(a[i] - want) <= 1e-4f * std::fabs(want);
    }
    expect(ok, "Allreduce(sum) in place");

    // non-blocking out-of-place allreduce (progress engine -> MPI_Iallreduce / MPI_Test)
    std::vector<float> s(n), r(n, -1.f);
    for (size_t i = 0; i < n; ++i) s[i] = val(me, i + 3);
    B::req_type req = B::null_req;
    Al::NonblockingAllreduce<B>(s.data(), r.data(), n, Al::ReductionOperator::max, comm, req);
    Al::Wait<B>(req);
    ok = true;
    for (size_t i = 0; i < n; ++i) ok = ok && r[i] == val(p - 1, i + 3);
    expect(ok, "NonblockingAllreduce(max) + Wait");

    // bcast
    std::vector<int> b(1000, me == p - 1 ? 7 : 0);
    if (me == p - 1) for (size_t i = 0; i < b.size(); ++i) b[i] = (int)i * 3;
    Al::Bcast<B>(b.data(), b.size(), p - 1, comm);
    ok = true;
    for (size_t i = 0; i < b.size(); ++i) ok = ok && b[i] == (int)i * 3;
    expect(ok, "Bcast");

    // alltoall
    const size_t m = 4096;
    std::vector<int> as(m * (size_t)p), ar(m * (size_t)p, -1);
    for (int d = 0; d < p; ++d)
      for (size_t i = 0; i < m; ++i) as[(size_t)d * m + i] = me * 1000000 + d * 10000 + (int)i;
    Al::Alltoall<B>(as.data(), ar.data(), m, comm);
    ok = true;
    for (int src = 0; src < p; ++src)
      for (size_t i = 0; i < m; ++i) ok = ok && ar[(size_t)src * m + i] == src * 1000000 + me * 10000 + (int)i;
    expect(ok, "Alltoall");

    // allgather, reduce_scatter
    std::vector<double> gs(257, (double)me + 0.5), gr(257 * (size_t)p, 0);
    Al::Allgather<B>(gs.data(), gr.data(), gs.size(), comm);
    ok = true;
    for (int src = 0; src < p; ++src)
      for (size_t i = 0; i < 257; ++i) ok = ok && gr[(size_t)src * 257 + i] == (double)src + 0.5;
    expect(ok, "Allgather");
    std::vector<long long> rs(33 * (size_t)p), rr(33, 0);
    for (size_t i = 0; i < rs.size(); ++i) rs[i] = (long long)(me + 1) * (long long)i;
    Al::Reduce_scatter<B>(rs.data(), rr.data(), 33, Al::ReductionOperator::sum, comm);
    ok = true;
    const long long tri = (long long)p * (p + 1) / 2;
    for (size_t i = 0; i < 33; ++i) ok = ok && rr[i] == tri * (long long)((size_t)me * 33 + i);
    expect(ok, "Reduce_scatter");

    // gather / scatter with root 0, reduce to root p-1
    std::vector<int> g1(5, me), g2(5 * (size_t)p, -1);
    Al::Gather<B>(g1.data(), g2.data(), 5, 0, comm);
    if (me == 0) {
      ok = true;
      for (int src = 0; src < p; ++src) for (int i = 0; i < 5; ++i) ok = ok && g2[(size_t)src * 5 + i] == src;
      expect(ok, "Gather");
    }
    std::vector<int> s1(3 * (size_t)p), s2(3, -1);
    for (size_t i = 0; i < s1.size(); ++i) s1[i] = (int)i;
    Al::Scatter<B>(s1.data(), s2.data(), 3, 0, comm);
    expect(s2[0] == me * 3 && s2[2] == me * 3 + 2, "Scatter");
    std::vector<float> r1(64, (float)(me + 1)), r2(64, 0.f);
    Al::Reduce<B>(r1.data(), r2.data(), 64, Al::ReductionOperator::prod, p - 1, comm);
    if (me == p - 1) {
      float f = 1;
      for (int k = 1; k <= p; ++k) f *= (float)k;
      expect(r2[0] == f && r2[63] == f, "Reduce(prod)");
    }

    // ring SendRecv on a copied communicator, then a barrier
    B::comm_type comm2 = comm.copy();
    std::vector<int> x(1 << 20, me), y(1 << 20, -1);   // 4 MiB each way: larger than the socket buffers
    Al::SendRecv<B>(x.data(), x.size(), (me + 1) % p, y.data(), y.size(), (me + p - 1) % p, comm2);
    expect(y[0] == (me + p - 1) % p && y.back() == (me + p - 1) % p, "SendRecv ring");
    Al::Barrier<B>(comm2);
  }
  Al::Finalize();
  if (g_fail == 0) printf("[rank %d] mpi_shim + reference MPI backend: ok\n", g_rank);
  return g_fail ? 1 : 0;
}
