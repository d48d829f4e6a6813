// Low-latency kernel for small uniform allreduce / reduce_scatter / allgather / alltoall.
//
// The staged protocol costs a small message three trips: data stores, a release fence that waits
// for their acknowledgement, and the flag store.  Here the flag travels inside the data: a rank
// writes 16-byte vectors {word, epoch, word, epoch} straight into the receiver's packet slot and
// the receiver polls those vectors until both epochs are the operation's.  One trip, no fence, no
// flag round, no copy into staging - the latency regime that the reference gets from NCCL's LL
// protocol behind ncclAllReduce / ncclReduceScatter / ncclAllGather / ncclSend+ncclRecv
// (include/aluminum/nccl_impl.hpp:951,1306,1193,1235-1244).
//
// Slots: [parity of the operation number][source rank], kLLSlotBytes each, in every rank's workspace.
// Two parities suffice because each of the four operations makes every rank wait for data from
// every rank: a rank that has finished operation k+1 knows that every peer has finished operation k,
// so the slots of k may be overwritten by k+2.  (Rooted and empty operations give no such guarantee
// and stay on the staged path, where every rank waits for every rank's flag.)
//
// Work is split by 16-byte payload "groups"; group g of every slice belongs to the same thread in
// the sending loop and in the receiving loop, which is what makes the in-place forms safe: a thread
// overwrites only elements it has already sent.  Reductions fold the ranks in rank order, so every
// rank computes bit-identical results.  Every poll is bounded.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"
#include "packets.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

template <typename T, typename Red>
__global__ void __launch_bounds__(256) ll_kernel(const __grid_constant__ LLParams P, Red red) {
  using A = typename Elem<T>::Acc;
  constexpr int VEC = 16 / (int)sizeof(T);
  const Workspace& ws = P.ws;
  const int p = ws.p;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;
  stamp(ws, 0);

  const DevColl kind = (DevColl)P.kind;
  const uint32_t flag = (uint32_t)P.seq | 1u;  // never 0 (fresh memory); distinct for the operations that share a parity
  const size_t par_off = (size_t)(P.seq & 1) * (size_t)kMaxRanks * kLLSlotBytes;
  const size_t n = P.count;
  const size_t groups = (n + VEC - 1) / VEC;
  const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, nthr = (size_t)gridDim.x * blockDim.x;
  const T* send = (const T*)P.send[rank];
  T* recv = (T*)P.recv[rank];
  char* my_slots = ws.ll[rank] + par_off;               // [source rank]
  const size_t to_me = par_off + (size_t)rank * kLLSlotBytes;  // my slot inside a peer's area

  if (P.two_phase) {
    // ---------------- two-phase allreduce ---------------------------------------------------------
    // Slice r (groups [r*per, (r+1)*per)) is reduced by rank r.  Phase 1: every rank sends its groups of slice d
    // to rank d (first half of the slot).  The owner folds the p contributions in rank order, keeps the result
    // and sends it to every peer (phase 2, second half of the owner's slot in every peer's area), which
    // copies it out.  Traffic per rank 2(p-1)/p of the vector instead of p-1 times the vector; a second
    // NVLink trip, but still no flag round and no fence.  Group g is handled by the same thread in every
    // loop, so an in-place call only overwrites elements its own thread has already sent.
    const size_t per = (groups + (size_t)p - 1) / (size_t)p;
    const size_t half_slot = kLLSlotBytes / 2;
    for (size_t g = tid; g < groups; g += nthr) {
      const int d = (int)(g / per);
      if (d != rank) send_group(ws.ll[d] + to_me, g - (size_t)d * per, load_group(send, g * VEC, n), flag);
    }
    stamp(ws, 1);
    const uint64_t epoch = make_epoch(P.seq, 1);
    bool first = true;
    const size_t mine_lo = (size_t)rank * per, mine_hi = mine_lo + per < groups ? mine_lo + per : groups;
    for (size_t g = tid; g < groups; g += nthr) {
      if (g < mine_lo || g >= mine_hi) continue;
      A acc[VEC];
      for (int r = 0; r < p; ++r) {
        union { uint4 u; T e[VEC]; } x;
        if (r == rank) x.u = load_group(send, g * VEC, n);
        else if (!recv_group(my_slots + (size_t)r * kLLSlotBytes, g - mine_lo, flag, x.u, ws, rank, r, epoch, P.timeout_ns)) return;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const A a = Elem<T>::up(x.e[k]);
          acc[k] = r == 0 ? a : red(acc[k], a);
        }
      }
      if (first) { stamp(ws, 2); first = false; }
      union { uint4 u; T e[VEC]; } o;
#pragma unroll
      for (int k = 0; k < VEC; ++k) o.e[k] = Elem<T>::down(finish_acc(acc[k], P.scale, P.int_div));
      for (int i = 1; i < p; ++i) {
        const int d = (rank + i) % p;
        send_group(ws.ll[d] + to_me + half_slot, g - mine_lo, o.u, flag);
      }
      store_group(recv, g * VEC, n, o.u);
    }
    const uint64_t epoch2 = make_epoch(P.seq, 2);
    for (size_t g = tid; g < groups; g += nthr) {
      const int owner = (int)(g / per);
      if (owner == rank) continue;
      uint4 v;
      if (!recv_group(my_slots + (size_t)owner * kLLSlotBytes + half_slot, g - (size_t)owner * per, flag, v, ws, rank, owner, epoch2, P.timeout_ns)) return;
      store_group(recv, g * VEC, n, v);
    }
    stamp(ws, 3);
    return;
  }

  // ---------------- send ----------------------------------------------------------------------
  for (size_t g = tid; g < groups; g += nthr) {
    if (kind == DevColl::allreduce || kind == DevColl::allgather) {
      const uint4 v = load_group(send, g * VEC, n);
      for (int i = 1; i < p; ++i) {
        const int d = (rank + i) % p;
        send_group(ws.ll[d] + to_me, g, v, flag);
      }
    } else {  // reduce_scatter / alltoall: slice d goes to rank d
      for (int i = 1; i < p; ++i) {
        const int d = (rank + i) % p;
        send_group(ws.ll[d] + to_me, g, load_group(send + (size_t)d * n, g * VEC, n), flag);
      }
    }
  }

  stamp(ws, 1);
  // ---------------- receive ---------------------------------------------------------------------
  const uint64_t epoch = make_epoch(P.seq, 1);
  bool first = true;
  for (size_t g = tid; g < groups; g += nthr) {
    if (kind == DevColl::allreduce || kind == DevColl::reduce_scatter) {
      const T* own = kind == DevColl::allreduce ? send : send + (size_t)rank * n;
      A acc[VEC];
      for (int r = 0; r < p; ++r) {
        union { uint4 u; T e[VEC]; } x;
        if (r == rank) x.u = load_group(own, g * VEC, n);
        else if (!recv_group(my_slots + (size_t)r * kLLSlotBytes, g, flag, x.u, ws, rank, r, epoch, P.timeout_ns)) return;
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const A a = Elem<T>::up(x.e[k]);
          acc[k] = r == 0 ? a : red(acc[k], a);
        }
      }
      if (first) { stamp(ws, 2); first = false; }
      union { uint4 u; T e[VEC]; } o;
#pragma unroll
      for (int k = 0; k < VEC; ++k) o.e[k] = Elem<T>::down(finish_acc(acc[k], P.scale, P.int_div));
      store_group(recv, g * VEC, n, o.u);
    } else {  // allgather / alltoall: slice r of the result comes from rank r
      const T* own = kind == DevColl::allgather ? send : send + (size_t)rank * n;
      for (int i = 0; i < p; ++i) {
        const int r = (rank + i) % p;
        uint4 v;
        if (r == rank) {
          if (own == recv + (size_t)rank * n) continue;  // in place: already there
          v = load_group(own, g * VEC, n);
        } else if (!recv_group(my_slots + (size_t)r * kLLSlotBytes, g, flag, v, ws, rank, r, epoch, P.timeout_ns)) {
          return;
        }
        store_group(recv + (size_t)r * n, g * VEC, n, v);
      }
      if (first) { stamp(ws, 2); first = false; }
    }
  }
  stamp(ws, 3);
}

template <typename T, typename Red>
void do_launch(const LLParams& P, Red red, int ctas, int threads, int local_ranks, cudaStream_t stream) {
  void* args[] = {(void*)&P, (void*)&red};
  auto k = ll_kernel<T, Red>;
  const dim3 grid((unsigned)ctas, (unsigned)local_ranks, 1);
  if (local_ranks > 1)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)k, grid, dim3((unsigned)threads), args, 0, stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)k, grid, dim3((unsigned)threads), args, 0, stream));
}

template <typename T>
void launch_typed(const LLParams& P, int ctas, int threads, int local_ranks, cudaStream_t s) {
  switch ((ReductionOperator)P.op) {
    case ReductionOperator::sum:
    case ReductionOperator::avg: return do_launch<T>(P, RedSum(), ctas, threads, local_ranks, s);
    case ReductionOperator::min: return do_launch<T>(P, RedMin(), ctas, threads, local_ranks, s);
    case ReductionOperator::max: return do_launch<T>(P, RedMax(), ctas, threads, local_ranks, s);
    default: return do_launch<T>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
  }
}

bool is_int(DType t) {
  switch (t) {
    case DType::i8: case DType::u8: case DType::i16: case DType::u16:
    case DType::i32: case DType::u32: case DType::i64: case DType::u64: return true;
    default: return false;
  }
}

}  // namespace

bool ll_supported(DevColl kind, DType dt, ReductionOperator op) {
  if (kind == DevColl::allgather || kind == DevColl::alltoall) return dt == DType::u8;
  if (kind != DevColl::allreduce && kind != DevColl::reduce_scatter) return false;
  const bool bitwise = op == ReductionOperator::bor || op == ReductionOperator::band || op == ReductionOperator::bxor;
  if (is_int(dt)) return true;
  if (dt == DType::f32 || dt == DType::f64 || dt == DType::f16 || dt == DType::bf16) return !bitwise;
  return false;
}

void launch_ll(const LLParams& P, DType dt, int ctas, int threads, int local_ranks, cudaStream_t s) {
  const DevColl kind = (DevColl)P.kind;
  if (kind == DevColl::allgather || kind == DevColl::alltoall)
    return do_launch<uint8_t>(P, RedNone(), ctas, threads, local_ranks, s);
  switch (dt) {
    case DType::f32: return launch_typed<float>(P, ctas, threads, local_ranks, s);
    case DType::f64: return launch_typed<double>(P, ctas, threads, local_ranks, s);
    case DType::f16: return launch_typed<__half>(P, ctas, threads, local_ranks, s);
    case DType::bf16: return launch_typed<__nv_bfloat16>(P, ctas, threads, local_ranks, s);
    case DType::i8: return do_launch<int8_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    case DType::u8: return do_launch<uint8_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    case DType::i16: return do_launch<int16_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    case DType::u16: return do_launch<uint16_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    case DType::i32: return do_launch<int32_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    case DType::u32: return do_launch<uint32_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    case DType::i64: return do_launch<int64_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    case DType::u64: return do_launch<uint64_t>(P, RedRuntime{P.op}, ctas, threads, local_ranks, s);
    default: throw_al_exception("low-latency kernel: datatype not supported");
  }
}

}  // namespace device
}  // namespace internal
}  // namespace Al
