// Row exchange: alltoall(v) of rows that are strided or index-selected in the user's tensors, with the
// pack and unpack fused into the publish and consume steps (see RowsParams in al/device/params.hpp).
//
// It is the generic staged protocol - push into slot [me] of the destination's staging half, epoch
// handshake on the A flags, local consume, chunked over rows when a slice exceeds a slot, closing
// C barrier after a multi-chunk launch - with one warp per row instead of a flat byte range.  Uses:
// sequence <-> head transposition (Ulysses attention) and token dispatch / combine by expert without a
// permute().contiguous() or index_select copy before or after the alltoall.  The reference would need
// a pack kernel, ncclSend / ncclRecv groups and an unpack kernel (include/aluminum/nccl_impl.hpp:1251-1296).
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

__device__ __forceinline__ size_t rows_in_chunk(size_t rows, uint64_t c, size_t per_chunk) {
  const size_t lo = (size_t)c * per_chunk;
  if (rows <= lo) return 0;
  return rows - lo < per_chunk ? rows - lo : per_chunk;
}

__global__ void __launch_bounds__(512) rows_kernel(const __grid_constant__ RowsParams P) {
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;
  const uint64_t my_proto = proto_word(kProtoStaged, (int)DevColl::alltoall, 4);
  if (blockIdx.x == 0) post_entered(ws, rank, P.seq, my_proto, 0, 0);

  const RowTable& T = P.tab[rank];
  const size_t half = ws.half_bytes;
  const size_t cap_b = (half / (size_t)p) / 256 * 256;
  const size_t rb = P.row_bytes;
  const size_t per_chunk = cap_b / rb;  // rows of one slice that fit a slot (the host made sure it is >= 1)
  const char* send = (const char*)P.send[rank];
  char* recv = (char*)P.recv[rank];
  const long long* sidx = P.send_idx[rank];
  const long long* ridx = P.recv_idx[rank];
  const unsigned lane = threadIdx.x & 31;
  const size_t warp = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const size_t nwarps = (size_t)gridDim.x * (blockDim.x >> 5);

  __shared__ uint64_t s_chunks;
  uint64_t G = P.local_chunks[rank];
  for (uint64_t c = 0; c < G; ++c) {
    const size_t par_off = (size_t)((P.seq + c) & 1) * half;
    // ---- publish: row k of the slice for rank d -> d's slot [me], packed ----------------------------
    for (int i = 0; i < p; ++i) {
      const int d = (rank + 1 + i) % p;
      const size_t n = rows_in_chunk(T.send_rows[d], c, per_chunk);
      char* slot = ws.stage[d] + par_off + (size_t)rank * cap_b;
      for (size_t k = warp; k < n; k += nwarps) {
        size_t id = T.send_first[d] + (size_t)c * per_chunk + k;
        if (sidx) id = (size_t)sidx[id];
        group_copy(slot + k * rb, send + T.send_peer_off[d] + id * P.send_row_stride, rb, false, lane, 32);
      }
    }
    const uint64_t e = make_epoch(P.seq, c + 1);
    arrive_and_post(ws, rank, FlagLayout::off_A, 0, gridDim.x, e, c == 0, (int)(P.seq & 1), P.local_chunks[rank], my_proto);
    if (!wait_all(ws, rank, FlagLayout::off_A, 0, e, P.timeout_ns)) return;
    if (c == 0) {
      if (p > 1 && !protocols_agree(ws, rank, P.seq, my_proto)) return;
      if (threadIdx.x == 0) {
        uint64_t g = 1;
        for (int r = 0; r < p; ++r) {
          const uint64_t m = ld_relaxed_sys(flag_slot(ws.flags[rank], FlagLayout::off_meta, (int)(P.seq & 1) * kMaxRanks + r) + kMetaChunks);
          g = m > g ? m : g;
        }
        s_chunks = g;
      }
      __syncthreads();
      G = s_chunks;
    }
    // ---- consume: my slot [r] -> row k of what rank r sent me ------------------------------------------
    const char* mystage = ws.stage[rank] + par_off;
    for (int r = 0; r < p; ++r) {
      const size_t n = rows_in_chunk(T.recv_rows[r], c, per_chunk);
      const char* slot = mystage + (size_t)r * cap_b;
      for (size_t k = warp; k < n; k += nwarps) {
        size_t id = T.recv_first[r] + (size_t)c * per_chunk + k;
        if (ridx) id = (size_t)ridx[id];
        group_copy(recv + T.recv_peer_off[r] + id * P.recv_row_stride, slot + k * rb, rb, true, lane, 32);
      }
    }
  }
  if (G > 1) {
    const uint64_t e = make_epoch(P.seq, 1);
    arrive_and_post(ws, rank, FlagLayout::off_C, 2, gridDim.x, e, false, 0, 0);
    (void)wait_all(ws, rank, FlagLayout::off_C, 2, e, P.timeout_ns);
  }
}

}  // namespace

void launch_rows(const RowsParams& P, int ctas, int threads, int local_ranks, cudaStream_t stream) {
  void* args[] = {(void*)&P};
  const dim3 grid((unsigned)ctas, (unsigned)local_ranks, 1);
  if (local_ranks > 1)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)rows_kernel, grid, dim3((unsigned)threads), args, 0, stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)rows_kernel, grid, dim3((unsigned)threads), args, 0, stream));
}

}  // namespace device
}  // namespace internal
}  // namespace Al
