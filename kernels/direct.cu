// Allgather / alltoall straight into the peers' receive buffers.
//
// When every rank's receive buffer lives in symmetric memory (same offset of the
// same symm_alloc() block on every rank) nothing has to be staged: a rank stores
// its contribution at its final place in every destination's buffer over NVLink,
// and two flag rounds frame the operation -
//   A: "I have entered the operation": the stream order of the poster guarantees
//      that its earlier work on the receive buffer is complete, so peers may now
//      overwrite it;
//   B: "all my stores are performed": once a rank holds B from everyone its own
//      receive buffer is complete.
// No staging half is touched and there are no chunks, so the message size is
// not limited by the staging area and HBM sees each byte once on each side.
//
// Bulk = false moves the data with the CTA-wide store loops of datamove.cuh;
// Bulk = true lets one thread per CTA drive the bulk copy engine (bulk_copy.cuh),
// loading each tile of the local send buffer once and storing it to every
// destination.  Every load reads this GPU's own memory.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "bulk_copy.cuh"
#include "bulk_tiles.cuh"
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

constexpr int kBufs = 4;
constexpr int kTile = 32768;
constexpr size_t kSmem = (size_t)kBufs * kTile + 128;

template <bool Bulk>
__global__ void __launch_bounds__(512) direct_kernel(const __grid_constant__ CollParams P) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ int s_fail;
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;

  const DevColl kind = (DevColl)P.kind;
  const size_t count = P.tab[rank].send_counts[0];  // bytes per rank slice
  const char* send = (const char*)P.send[rank];
  const unsigned cta = blockIdx.x, nct = gridDim.x;
  const uint64_t e = make_epoch(P.seq, 1);

  bulk::Ring<kBufs, kTile> ring;
  if (threadIdx.x == 0) s_fail = 0;
  if (Bulk && threadIdx.x == 0) ring.init(dyn_smem, dyn_smem + (size_t)kBufs * kTile);

  // A: every rank has entered; its receive buffer may be written.
  arrive_and_post(ws, rank, FlagLayout::off_A, 0, nct, e, false, 0, 0);
  if (!wait_all(ws, rank, FlagLayout::off_A, 0, e, P.timeout_ns)) return;

  const plan::Share sh = plan::share_of(count, count, 0, cta, nct, kTile);  // one "chunk": the whole slice
  bool ok = true;
  if (send && sh.seg) {
    if (kind == DevColl::allgather) {
      // destinations rotated so that the ranks never converge on one ingress link; the own
      // buffer comes last and is skipped when the contribution already sits in place
      char* dsts[kMaxRanks];
      int n = 0;
#pragma unroll
      for (int i = 0; i < kMaxRanks; ++i) {
        dsts[i] = nullptr;
        if (i < p) {
          const int d = (rank + 1 + i) % p;
          char* base = (char*)P.recv[d];
          if (d == rank && base + (size_t)rank * count == send) continue;
          dsts[n++] = base;
        }
      }
      if constexpr (Bulk) {
        if (threadIdx.x == 0) {
          ok = bulk::stream_tiles(ring, sh.tiles, [&](size_t t, bulk::Tile& tl) {
            const plan::Move m = plan::ag_direct(sh, t, rank, count, kTile);
            tl.src = send + m.src;
            tl.bytes = m.bytes;
            tl.ndst = n;
            for (int i = 0; i < n; ++i) tl.dst[i] = dsts[i] + m.dst;
          }, P.timeout_ns);
          __threadfence_system();
        }
      } else {
        const plan::Move m = plan::ag_direct(sh, 0, rank, count, kTile);  // offsets of the share's first byte
        cta_fanout(dsts, n, m.dst, send + m.src, sh.seg);
      }
    } else {  // alltoall: slice d of the send buffer goes to rank d
      if constexpr (Bulk) {
        if (threadIdx.x == 0) {
          ok = bulk::stream_tiles(ring, plan::fan_tiles(sh, p), [&](size_t t, bulk::Tile& tl) {
            const plan::Move m = plan::a2a_direct(sh, t, rank, p, count, kTile);
            tl.src = send + m.src;
            tl.bytes = m.bytes;
            tl.ndst = 1;
            tl.dst[0] = (char*)P.recv[m.peer] + m.dst;
          }, P.timeout_ns);
          __threadfence_system();
        }
      } else {
        for (int i = 0; i < p; ++i) {
          const plan::Move m = plan::a2a_direct(sh, (size_t)i, rank, p, count, kTile);  // tile 0 towards destination i
          char* dst = (char*)P.recv[m.peer];
          cta_fanout(&dst, 1, m.dst, send + m.src, sh.seg);
        }
      }
    }
  }
  if constexpr (Bulk) {
    if (threadIdx.x == 0 && !ok) s_fail = 1;
    __syncthreads();
    if (s_fail) {
      if (threadIdx.x == 0) report_timeout(ws, rank, rank, 6, e, 0);
      return;
    }
  }
  // B: my stores are performed; with B from everyone my receive buffer is complete.
  arrive_and_post(ws, rank, FlagLayout::off_B, 1, nct, e, false, 0, 0);
  (void)wait_all(ws, rank, FlagLayout::off_B, 1, e, P.timeout_ns);
}

template <bool Bulk>
void launch_one(const CollParams& P, int ctas, int threads, int local_ranks, cudaStream_t stream) {
  auto k = direct_kernel<Bulk>;
  const size_t smem = Bulk ? kSmem : 0;
  if (Bulk) AL_CHECK_CUDA(cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
  void* args[] = {(void*)&P};
  const dim3 grid((unsigned)ctas, (unsigned)local_ranks, 1);
  if (local_ranks > 1)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)k, grid, dim3((unsigned)threads), args, smem, stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)k, grid, dim3((unsigned)threads), args, smem, stream));
}

}  // namespace

void launch_direct(const CollParams& P, bool bulk_engine, int ctas, int threads, int local_ranks, cudaStream_t stream) {
  const DevColl kind = (DevColl)P.kind;
  if (kind != DevColl::allgather && kind != DevColl::alltoall)
    throw_al_exception("direct kernel: only allgather and alltoall");
  if (bulk_engine) launch_one<true>(P, ctas, threads, local_ranks, stream);
  else launch_one<false>(P, ctas, threads, local_ranks, stream);
}

}  // namespace device
}  // namespace internal
}  // namespace Al
