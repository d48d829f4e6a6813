// Window kernels: uniform reduce_scatter / allgather / alltoall / bcast that work straight on
// registered buffers ("windows": memory every rank of the communicator can address, see
// DeviceCommunicator::register_buffer and symm_alloc) - no staging area, no chunks, no copy-out.
//
//   allgather / alltoall / bcast   the RECEIVE buffers are registered: a rank stores its contribution at
//                                  its final place in every destination's buffer (peer stores over NVLink, or
//                                  one multimem.st that the NVSwitch replicates when all receive buffers are
//                                  the same offset of one multicast-bound window);
//   reduce_scatter                 the SEND buffers are registered: a rank reduces its slice out of every
//                                  rank's send buffer (peer loads folded in rank order, or one
//                                  multimem.ld_reduce that the NVSwitch reduces) into its private or
//                                  registered receive buffer, with the scale / average fused in.
//
// Role: what ncclAllGather / ncclReduceScatter / ncclBroadcast / grouped ncclSend+ncclRecv do for the
// reference on registered buffers (include/aluminum/nccl_impl.hpp:1096,1193,1235-1244,1306 with
// src/nccl_impl.cpp:83-109).
//
// Protocol (flags B and C of the communicator, epoch = operation number):
//   B  "entered", carrying the protocol word and the descriptors (window, offset) of this rank's
//      buffers: the poster's earlier work on its buffers is complete, peers may touch them; every
//      rank learns where every rank's buffer of THIS call lies, so offsets may differ between ranks;
//   -- data movement --
//   C  "done": my stores are performed / I have read all I need; with C from everyone a rank's
//      receive buffer is complete and its send buffer may be reused.
// A rank that entered the same operation through the staging kernels announces that in its B word;
// both sides then stop with a kStatusMismatch record instead of a time-out (common.cuh, protocols_agree).
// Every wait is bounded.  No TMA, no cluster-multicast load: remote data moves with ordinary loads
// and stores and multimem instructions only.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"
#include "multimem.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

__device__ __forceinline__ int win_of(uint64_t desc) { return (int)(desc >> 48) - 1; }
__device__ __forceinline__ size_t off_of(uint64_t desc) { return (size_t)(desc & ((uint64_t{1} << 48) - 1)); }

struct Descs {
  uint64_t recv[kMaxRanks];
  uint64_t send[kMaxRanks];
};

/** Entered round + protocol comparison + descriptor fetch.  Block-uniform; false = give up. */
__device__ __forceinline__ bool enter_operation(const WinParams& P, int rank, Descs& sh) {
  const Workspace& ws = P.ws;
  const uint64_t mine = proto_word(kProtoWindow, P.kind);
  if (blockIdx.x == 0) post_entered(ws, rank, P.seq, mine, P.recv_desc[rank], P.send_desc[rank]);
  if (!wait_all(ws, rank, FlagLayout::off_B, 1, make_epoch(P.seq, 1), P.timeout_ns)) return false;
  if (!protocols_agree(ws, rank, P.seq, mine)) return false;
  if (threadIdx.x < ws.p) {
    const uint64_t* m = flag_slot(ws.flags[rank], FlagLayout::off_meta, (int)(P.seq & 1) * kMaxRanks + threadIdx.x);
    sh.recv[threadIdx.x] = ld_relaxed_sys(m + kMetaRecvDesc);
    sh.send[threadIdx.x] = ld_relaxed_sys(m + kMetaSendDesc);
  }
  __syncthreads();
  return true;
}

__device__ __forceinline__ void leave_operation(const WinParams& P, int rank) {
  __threadfence_system();
  arrive_and_post(P.ws, rank, FlagLayout::off_C, 2, gridDim.x, make_epoch(P.seq, 1), false, 0, 0);
  (void)wait_all(P.ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, 1), P.timeout_ns);
}

/** Address, in this process, of rank r's buffer described by `desc` (the own buffer is `local`). */
__device__ __forceinline__ char* window_addr(const WindowTable* W, uint64_t desc, int r, int me, const void* local) {
  if (r == me) return (char*)local;
  return W->peer[win_of(desc)][r] + off_of(desc);
}

/** All descriptors equal (same window, same offset): the condition for one multicast address. */
__device__ __forceinline__ bool all_same(const uint64_t* d, int p) {
  bool same = true;
  for (int r = 1; r < p; ++r) same = same && d[r] == d[0];
  return same;
}

/** Replicate the 16-byte vectors [0, nvec) of `src` to the multicast address, this CTA's share. */
__device__ __forceinline__ void multicast_copy(char* mc_dst, const char* src, size_t nvec, unsigned part, unsigned nparts) {
  const size_t stride = (size_t)blockDim.x * nparts;
  size_t v = (size_t)part * blockDim.x + threadIdx.x;
  const uint4* s = (const uint4*)src;
  for (; v + 3 * stride < nvec; v += 4 * stride) {
    const uint4 a = s[v], b = s[v + stride], c = s[v + 2 * stride], d = s[v + 3 * stride];
    mm_st(mc_dst + (v << 4), a);
    mm_st(mc_dst + ((v + stride) << 4), b);
    mm_st(mc_dst + ((v + 2 * stride) << 4), c);
    mm_st(mc_dst + ((v + 3 * stride) << 4), d);
  }
  for (; v < nvec; v += stride) mm_st(mc_dst + (v << 4), s[v]);
}

/**
 * Copy [0, n) of `src` to every destination.  When source and destinations are 16-byte aligned the vectors
 * are stored to all destinations in turn (every link and the local memory stay busy at the same time);
 * otherwise one destination after the other with whatever width the alignment allows.
 */
__device__ __forceinline__ void fan_copy(char* const* dsts, int ndst, const char* src, size_t n) {
  if (n == 0 || ndst == 0) return;
  uintptr_t mis = (uintptr_t)src | (uintptr_t)n;
  for (int d = 0; d < ndst; ++d) mis |= (uintptr_t)dsts[d];
  if ((mis & 15) == 0) {
    const uint4* s = (const uint4*)src;
    const size_t nv = n >> 4, stride = blockDim.x;
    size_t i = threadIdx.x;
    for (; i + 3 * stride < nv; i += 4 * stride) {
      const uint4 a = s[i], b = s[i + stride], c = s[i + 2 * stride], e = s[i + 3 * stride];
#pragma unroll
      for (int d = 0; d < kMaxRanks; ++d) {
        if (d < ndst) {
          uint4* o = (uint4*)dsts[d];
          o[i] = a; o[i + stride] = b; o[i + 2 * stride] = c; o[i + 3 * stride] = e;
        }
      }
    }
    for (; i < nv; i += stride) {
      const uint4 a = s[i];
#pragma unroll
      for (int d = 0; d < kMaxRanks; ++d)
        if (d < ndst) ((uint4*)dsts[d])[i] = a;
    }
    return;
  }
  for (int d = 0; d < ndst; ++d) cta_copy(dsts[d], src, n, false);
}

// ---------------------------------------------------------------------------------------------
// allgather / alltoall / bcast: byte movement into registered receive buffers
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(512) window_move_kernel(const __grid_constant__ WinParams P) {
  __shared__ Descs sh;
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;
  if (!enter_operation(P, rank, sh)) return;

  const DevColl kind = (DevColl)P.kind;
  const size_t count = P.count;  // bytes per slice
  const char* send = (const char*)P.send[rank];
  char* recv = (char*)P.recv[rank];
  const WindowTable* W = P.windows;
  const unsigned cta = blockIdx.x, nct = gridDim.x;

  // One multicast address reaches every receive buffer when they are the same offset of one multicast-bound window.
  char* mc = nullptr;
  if (P.allow_multimem && all_same(sh.recv, p) && sh.recv[0] != 0) {
    char* base = W->mc[win_of(sh.recv[0])];
    if (base) mc = base + off_of(sh.recv[0]);
  }
  const bool vec_ok = count % 16 == 0 && ((uintptr_t)send & 15) == 0 && mc != nullptr && ((uintptr_t)mc & 15) == 0;

  if (kind == DevColl::allgather) {
    if (send && count) {
      // A multicast store also comes back to its sender: p slices enter every GPU instead of p-1.  The host
      // allows it for allgather (bit 1) only where saving p-2 store instructions per vector is worth that.
      if (vec_ok && (P.allow_multimem & 2)) {
        // the switch delivers the slice to every rank, this one included
        multicast_copy(mc + (size_t)rank * count, send, count >> 4, cta, nct);
      } else {
        size_t lo, hi;
        split_range(count, cta, nct, 16, lo, hi);
        char* dsts[kMaxRanks];
        int n = 0;
#pragma unroll
        for (int i = 0; i < kMaxRanks; ++i) {
          dsts[i] = nullptr;
          if (i < p) {
            const int d = (rank + 1 + i) % p;  // rotated: the ranks start on distinct peers
            char* dst = window_addr(W, sh.recv[d], d, rank, recv) + (size_t)rank * count;
            if (!(d == rank && dst == send)) dsts[n++] = dst + lo;  // in place: the contribution already sits there
          }
        }
        if (hi > lo) fan_copy(dsts, n, send + lo, hi - lo);
      }
    }
  } else if (kind == DevColl::alltoall) {
    if (send && count) {
      size_t lo, hi;
      split_range(count, cta, nct, 16, lo, hi);
      for (int i = 0; i < p && hi > lo; ++i) {
        const int d = (rank + 1 + i) % p;
        char* dst = window_addr(W, sh.recv[d], d, rank, recv) + (size_t)rank * count;
        cta_copy(dst + lo, send + (size_t)d * count + lo, hi - lo, false);
      }
    }
  } else if (kind == DevColl::bcast) {
    if (rank == P.root && send && count) {
      if (vec_ok) {
        multicast_copy(mc, send, count >> 4, cta, nct);  // rewrites the root's own buffer with the same bytes
      } else {
        size_t lo, hi;
        split_range(count, cta, nct, 16, lo, hi);
        char* dsts[kMaxRanks];
        int n = 0;
#pragma unroll
        for (int i = 0; i < kMaxRanks; ++i) {
          dsts[i] = nullptr;
          if (i < p - 1) dsts[n++] = window_addr(W, sh.recv[(rank + 1 + i) % p], (rank + 1 + i) % p, rank, recv) + lo;
        }
        if (hi > lo) fan_copy(dsts, n, send + lo, hi - lo);
      }
    }
  }
  leave_operation(P, rank);
}

// ---------------------------------------------------------------------------------------------
// reduce_scatter out of registered send buffers
// ---------------------------------------------------------------------------------------------
template <typename T, NvOp OP, bool HasMM>
struct SwitchLoad {
  static __device__ __forceinline__ uint4 ld(const void*) { return uint4{0, 0, 0, 0}; }
};
template <typename T, NvOp OP>
struct SwitchLoad<T, OP, true> {
  static __device__ __forceinline__ uint4 ld(const void* mc) { return MM<T, OP>::ld(mc); }
};

template <typename T, typename Red, NvOp OP, bool HasMM>
__global__ void __launch_bounds__(512) window_reduce_kernel(const __grid_constant__ WinParams P, Red red) {
  __shared__ Descs sh;
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;
  if (!enter_operation(P, rank, sh)) return;

  const size_t count = P.count;  // elements this rank receives
  T* recv = (T*)P.recv[rank];
  const WindowTable* W = P.windows;
  const unsigned cta = blockIdx.x, nct = gridDim.x;
  constexpr size_t VEC = 16 / sizeof(T);

  char* mc = nullptr;
  if (HasMM && P.allow_multimem && all_same(sh.send, p) && sh.send[0] != 0) {
    char* base = W->mc[win_of(sh.send[0])];
    if (base) mc = base + off_of(sh.send[0]) + (size_t)rank * count * sizeof(T);
  }
  if (recv && count) {
    if (HasMM && mc && ((uintptr_t)mc & 15) == 0 && ((uintptr_t)recv & 15) == 0 && count % VEC == 0) {
      // the switch fetches the 16 bytes from every rank, reduces them and returns one result
      const size_t nvec = count / VEC;
      const size_t stride = (size_t)blockDim.x * nct;
      const float scale = (float)P.scale;
      uint4* out = (uint4*)recv;
      size_t v = (size_t)cta * blockDim.x + threadIdx.x;
      constexpr int U = 4;
      for (; v + (U - 1) * stride < nvec; v += U * stride) {
        uint4 a[U];
#pragma unroll
        for (int u = 0; u < U; ++u) a[u] = SwitchLoad<T, OP, HasMM>::ld(mc + ((v + u * stride) << 4));
#pragma unroll
        for (int u = 0; u < U; ++u) out[v + u * stride] = scale != 1.f ? scale_pack<T>(a[u], scale) : a[u];
      }
      for (; v < nvec; v += stride) {
        const uint4 a = SwitchLoad<T, OP, HasMM>::ld(mc + (v << 4));
        out[v] = scale != 1.f ? scale_pack<T>(a, scale) : a;
      }
    } else {
      char* bases[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        bases[r] = r < p ? window_addr(W, sh.send[r], r, rank, P.send[rank]) + (size_t)rank * count * sizeof(T) : nullptr;
      size_t lo, hi;
      split_range(count, cta, nct, VEC, lo, hi);
      if (hi > lo) {
        T* out = recv + lo;
        cta_reduce<T, T, Red>(&out, 1, bases, lo * sizeof(T), p, hi - lo, red, P.scale, P.int_div);
      }
    }
  }
  leave_operation(P, rank);
}

template <typename K, typename... Extra>
void launch_kernel(K kernel, const WinParams& P, int ctas, int threads, int local_ranks, cudaStream_t stream,
                   Extra... extra) {
  void* args[] = {(void*)&P, (void*)&extra...};
  const dim3 grid((unsigned)ctas, (unsigned)local_ranks, 1);
  if (local_ranks > 1)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)kernel, grid, dim3((unsigned)threads), args, 0, stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)kernel, grid, dim3((unsigned)threads), args, 0, stream));
}

template <typename T, bool MMAdd, bool MMMinMax>
void launch_reduce(const WinParams& P, ReductionOperator op, int ctas, int threads, int local_ranks, cudaStream_t s) {
  switch (op) {
    case ReductionOperator::sum:
    case ReductionOperator::avg:
      return launch_kernel(window_reduce_kernel<T, RedSum, NvOp::add, MMAdd>, P, ctas, threads, local_ranks, s, RedSum());
    case ReductionOperator::min:
      return launch_kernel(window_reduce_kernel<T, RedMin, NvOp::min, MMMinMax>, P, ctas, threads, local_ranks, s, RedMin());
    case ReductionOperator::max:
      return launch_kernel(window_reduce_kernel<T, RedMax, NvOp::max, MMMinMax>, P, ctas, threads, local_ranks, s, RedMax());
    default: throw_al_exception("window reduce_scatter: operator not supported");
  }
}

}  // namespace

bool window_supported(DevColl kind, DType dt, ReductionOperator op) {
  if (kind == DevColl::allgather || kind == DevColl::alltoall || kind == DevColl::bcast) return true;
  if (kind != DevColl::reduce_scatter) return false;
  if (dt != DType::f32 && dt != DType::f16 && dt != DType::bf16) return false;
  return op == ReductionOperator::sum || op == ReductionOperator::avg || op == ReductionOperator::min ||
         op == ReductionOperator::max;
}

void launch_window(const WinParams& P, DType dt, ReductionOperator op, int ctas, int threads, int local_ranks,
                   cudaStream_t stream) {
  const DevColl kind = (DevColl)P.kind;
  if (!window_supported(kind, dt, op)) throw_al_exception("window kernel: operation / type / operator not supported");
  if (kind != DevColl::reduce_scatter) return launch_kernel(window_move_kernel, P, ctas, threads, local_ranks, stream);
  if (dt == DType::f32) return launch_reduce<float, true, false>(P, op, ctas, threads, local_ranks, stream);
  if (dt == DType::bf16) return launch_reduce<__nv_bfloat16, true, true>(P, op, ctas, threads, local_ranks, stream);
  return launch_reduce<__half, true, true>(P, op, ctas, threads, local_ranks, stream);
}

}  // namespace device
}  // namespace internal
}  // namespace Al
