// Large uniform allgather / alltoall / reduce_scatter with the data moved by the
// bulk copy engine instead of SM load/store loops.
//
// Same protocol, staging layout, flags and epochs as the pipelined schedule of
// the generic collective kernel (coll_kernel.cuh), so ranks that pick different
// kernels for one operation (a rank whose buffers are not 16-byte aligned falls
// back to the generic kernel) still interoperate.  The lower `n_pub` CTAs
// publish: one thread per CTA streams tiles of this rank's send buffer through
// shared memory into slot [me] of the destination ranks' staging halves
// (cp.async.bulk global->shared, then shared->global over NVLink; an allgather
// tile is loaded once and stored to every rank).  The other CTAs consume:
// allgather / alltoall copy the p slots of the own staging half into the receive
// buffer with the same engine, reduce_scatter folds them with SM loads.
// The SMs only issue descriptors, so a handful of CTAs saturates the links and
// the rest of the GPU stays free for the application's kernels.
//
// Every load in this file reads this GPU's own memory and has exactly one destination CTA.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "bulk_copy.cuh"
#include "bulk_tiles.cuh"
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

constexpr int kBulkBufs = 4;
constexpr int kBulkTile = 32768;
constexpr size_t kBulkSmem = (size_t)kBulkBufs * kBulkTile + 128;  // tiles + barriers

template <typename T, typename Red>
__global__ void __launch_bounds__(512) bulk_pipeline_kernel(const __grid_constant__ CollParams P, Red red) {
  extern __shared__ __align__(128) unsigned char dyn_smem[];
  __shared__ int s_fail;
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;
  // same protocol (and the same announcement) as the pipelined schedule of the generic kernel
  const uint64_t my_proto = proto_word(kProtoStaged, P.kind, P.two_phase | (P.pipelined << 1));
  if (blockIdx.x == 0) post_entered(ws, rank, P.seq, my_proto, 0, 0);

  const DevColl kind = (DevColl)P.kind;
  const CountTable& Tb = P.tab[rank];
  const size_t half = ws.half_bytes;
  const size_t cap_b = (half / (size_t)p) / 256 * 256;  // one slot per source rank
  const size_t slot_e = P.slot_elems;                   // elements per slot and chunk (bytes * 1/sizeof(T) multiple of 16 bytes)
  constexpr size_t VEC = 16 / sizeof(T);
  const char* send = (const char*)P.send[rank];
  char* recv = (char*)P.recv[rank];
  const size_t count = Tb.send_counts[0];               // uniform: elements per rank slice
  const size_t slice_b = count * sizeof(T), slot_b = slot_e * sizeof(T);
  const uint64_t G = P.local_chunks[rank];
  const unsigned n_pub = P.n_pub > 0 ? (unsigned)P.n_pub : gridDim.x / 2;
  const unsigned n_con = gridDim.x - n_pub;

  bulk::Ring<kBulkBufs, kBulkTile> ring;
  if (threadIdx.x == 0) {
    ring.init(dyn_smem, dyn_smem + (size_t)kBulkBufs * kBulkTile);
    s_fail = 0;
  }
  __syncthreads();

  // Block-uniform outcome of a stage driven by thread 0.
  auto stage_failed = [&](bool ok, uint32_t where, uint64_t c) {
    if (threadIdx.x == 0 && !ok) s_fail = 1;
    __syncthreads();
    if (s_fail) {
      if (threadIdx.x == 0) report_timeout(ws, rank, rank, where, make_epoch(P.seq, c + 1), 0);
      return true;
    }
    return false;
  };

  if (blockIdx.x < n_pub) {
    // ------------------------------- publishers --------------------------------
    for (uint64_t c = 0; c < G; ++c) {
      if (c >= 2 && !wait_all(ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, c - 1), P.timeout_ns)) return;
      const int par = (int)((P.seq + c) & 1);
      const plan::Share sh = plan::share_of(slice_b, slot_b, c, blockIdx.x, n_pub, kBulkTile);
      bool ok = true;
      if (threadIdx.x == 0 && send && sh.seg) {
        const size_t half_off = (size_t)par * half;
        if (kind == DevColl::allgather) {
          ok = bulk::stream_tiles(ring, sh.tiles, [&](size_t t, bulk::Tile& tl) {
            const plan::Move m = plan::ag_publish(sh, t, rank, cap_b, kBulkTile);
            tl.src = send + m.src;
            tl.bytes = m.bytes;
            tl.ndst = p;
            for (int i = 0; i < p; ++i) tl.dst[i] = ws.stage[(rank + 1 + i) % p] + half_off + m.dst;
          }, P.timeout_ns);
        } else {  // reduce_scatter / alltoall: slice d goes to rank d; tiles rotate over the destinations
          ok = bulk::stream_tiles(ring, plan::fan_tiles(sh, p), [&](size_t t, bulk::Tile& tl) {
            const plan::Move m = plan::scatter_publish(sh, t, rank, p, slice_b, cap_b, kBulkTile);
            tl.src = send + m.src;
            tl.bytes = m.bytes;
            tl.ndst = 1;
            tl.dst[0] = ws.stage[m.peer] + half_off + m.dst;
          }, P.timeout_ns);
        }
        __threadfence_system();
      }
      if (stage_failed(ok, 6, c)) return;
      arrive_and_post(ws, rank, FlagLayout::off_A, 0, n_pub, make_epoch(P.seq, c + 1), c == 0, (int)(P.seq & 1), G, my_proto);
    }
  } else {
    // ------------------------------- consumers ----------------------------------
    const unsigned part = blockIdx.x - n_pub;
    for (uint64_t c = 0; c < G; ++c) {
      if (!wait_all(ws, rank, FlagLayout::off_A, 0, make_epoch(P.seq, c + 1), P.timeout_ns)) return;
      if (c == 0 && !protocols_agree(ws, rank, P.seq, my_proto)) return;
      const int par = (int)((P.seq + c) & 1);
      char* mystage = ws.stage[rank] + (size_t)par * half;
      const size_t base = c * slot_e, len = clamp_len(count, base, slot_e);
      size_t lo, hi;
      split_range(len, part, n_con, VEC, lo, hi);
      bool ok = true;
      if (kind == DevColl::reduce_scatter) {
        if (recv && hi > lo) {
          char* slot[kMaxRanks];
#pragma unroll
          for (int r = 0; r < kMaxRanks; ++r) slot[r] = mystage + (size_t)r * cap_b;
          T* out = (T*)recv + base + lo;
          cta_reduce<T, T, Red>(&out, 1, slot, lo * sizeof(T), p, hi - lo, red, P.scale, P.int_div);
        }
      } else {
        const plan::Share sh = plan::share_of(slice_b, slot_b, c, part, n_con, kBulkTile);
        if (threadIdx.x == 0 && recv && sh.seg) {
          ok = bulk::stream_tiles(ring, plan::fan_tiles(sh, p), [&](size_t t, bulk::Tile& tl) {
            const plan::Move m = plan::gather_consume(sh, t, p, slice_b, cap_b, kBulkTile);
            tl.src = mystage + m.src;
            tl.bytes = m.bytes;
            tl.ndst = 1;
            tl.dst[0] = recv + m.dst;
          }, P.timeout_ns);
        }
      }
      if (stage_failed(ok, 6, c)) return;
      arrive_and_post(ws, rank, FlagLayout::off_C, 2, n_con, make_epoch(P.seq, c + 1), false, 0, 0);
    }
  }
  // Closing barrier: every peer has consumed every chunk, both halves are free.
  (void)wait_all(ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, G), P.timeout_ns);
}

template <typename T, typename Red>
void launch_one(const CollParams& P, Red red, int ctas, int threads, int local_ranks, cudaStream_t stream) {
  auto k = bulk_pipeline_kernel<T, Red>;
  AL_CHECK_CUDA(cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBulkSmem));
  void* args[] = {(void*)&P, (void*)&red};
  const dim3 grid((unsigned)ctas, (unsigned)local_ranks, 1);
  if (local_ranks > 1)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)k, grid, dim3((unsigned)threads), args, kBulkSmem, stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)k, grid, dim3((unsigned)threads), args, kBulkSmem, stream));
}

}  // namespace

bool bulk_pipeline_supported(DevColl kind, DType dt, ReductionOperator op) {
  if (kind == DevColl::allgather || kind == DevColl::alltoall) return dt == DType::u8;
  if (kind == DevColl::reduce_scatter)
    return (op == ReductionOperator::sum || op == ReductionOperator::avg) &&
           (dt == DType::f32 || dt == DType::bf16 || dt == DType::f16);
  return false;
}

void launch_bulk_pipeline(const CollParams& P, DType dt, int ctas, int threads, int local_ranks, cudaStream_t stream) {
  const DevColl kind = (DevColl)P.kind;
  if (!bulk_pipeline_supported(kind, dt, (ReductionOperator)P.op) || !P.pipelined || P.slot_elems == 0)
    throw_al_exception("bulk pipeline kernel: unsupported operation");
  if (kind != DevColl::reduce_scatter) return launch_one<unsigned char>(P, RedNone(), ctas, threads, local_ranks, stream);
  switch (dt) {
    case DType::f32: return launch_one<float>(P, RedSum(), ctas, threads, local_ranks, stream);
    case DType::bf16: return launch_one<__nv_bfloat16>(P, RedSum(), ctas, threads, local_ranks, stream);
    default: return launch_one<__half>(P, RedSum(), ctas, threads, local_ranks, stream);
  }
}

}  // namespace device
}  // namespace internal
}  // namespace Al
