// NVLS (NVLink SHARP) allreduce: the NVSwitch reduces and replicates.
//
// Each rank owns 1/p of the vector.  For its slice it issues
// multimem.ld_reduce on the multicast address - the switch fetches the 16
// bytes from every GPU bound to the multicast object, reduces them and
// returns one result - applies the scale, and writes the result back with
// multimem.st, which the switch replicates into every GPU's memory.  Per GPU
// the links carry about S(1+1/p) bytes instead of the 2S(p-1)/p of a
// peer-to-peer two-shot.
//
// Two flavours share the kernel:
//   staged     - user buffers are private: copy into the multicast-bound
//                staging half, reduce in place there, copy out;
//   zero-copy  - user buffers come from the library's symmetric allocator and
//                have their own multicast alias: no copies at all.
// No TMA is involved anywhere; remote data moves only through multimem
// instructions.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"
#include "multimem.cuh"
#include "packets.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

/**
 * Reduce-and-replicate the 16-byte vectors [v_lo, v_hi) of the multicast range.
 * Each thread keeps U switch reductions in flight before it stores, so that a
 * modest number of CTAs covers the NVLink latency-bandwidth product.
 */
template <typename T, NvOp OP>
__device__ __forceinline__ void reduce_vectors(const char* mc_in, char* mc_out, size_t v_lo, size_t v_hi,
                                               float scale, unsigned part, unsigned nparts) {
  constexpr int U = 4;
  const size_t stride = (size_t)blockDim.x * nparts;
  size_t v = v_lo + (size_t)part * blockDim.x + threadIdx.x;
  for (; v + (U - 1) * stride < v_hi; v += U * stride) {
    uint4 a[U];
#pragma unroll
    for (int u = 0; u < U; ++u) a[u] = MM<T, OP>::ld(mc_in + ((v + u * stride) << 4));
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (scale != 1.f) a[u] = scale_pack<T>(a[u], scale);
      mm_st(mc_out + ((v + u * stride) << 4), a[u]);
    }
  }
  for (; v < v_hi; v += stride) {
    uint4 a = MM<T, OP>::ld(mc_in + (v << 4));
    if (scale != 1.f) a = scale_pack<T>(a, scale);
    mm_st(mc_out + (v << 4), a);
  }
}

template <typename T, NvOp OP>
__global__ void __launch_bounds__(512) nvls_allreduce_kernel(const __grid_constant__ NvlsParams P) {
  const Workspace& ws = P.ws;
  const int p = ws.p, rank = P.rank;
  if (poisoned(ws, rank)) return;
  const float scale = (float)P.scale;

  if (P.mc_in != nullptr) {
    // ---- zero-copy: operate on the user's symmetric buffers --------------------
    const uint64_t e = make_epoch(P.seq, 1);
    // The choice between this flavour and the staged one depends on this rank's own buffers: compare.
    const uint64_t my_proto = proto_word(kProtoNvlsZeroCopy, (int)DevColl::allreduce);
    arrive_and_post(ws, rank, FlagLayout::off_A, 0, gridDim.x, e, true, (int)(P.seq & 1), 1, my_proto);
    if (!wait_all(ws, rank, FlagLayout::off_A, 0, e, P.timeout_ns)) return;
    if (!protocols_agree(ws, rank, P.seq, my_proto)) return;
    const size_t nvec = (P.count * sizeof(T) + 15) >> 4;  // a tail vector only ever covers the block's own padding
    size_t s_lo, s_hi;
    split_range(nvec, (unsigned)rank, (unsigned)p, 1, s_lo, s_hi);
    reduce_vectors<T, OP>(P.mc_in, P.mc_out, s_lo, s_hi, scale, blockIdx.x, gridDim.x);
    __threadfence_system();
    arrive_and_post(ws, rank, FlagLayout::off_B, 1, gridDim.x, e, false, 0, 0);
    (void)wait_all(ws, rank, FlagLayout::off_B, 1, e, P.timeout_ns);
    return;
  }

  // ---- staged ------------------------------------------------------------------
  const size_t half = ws.half_bytes;
  const size_t full_e = half / sizeof(T);
  const T* send = (const T*)P.send;
  T* recv = (T*)P.recv;
  const uint64_t G = P.chunks;
  const uint64_t my_proto = proto_word(kProtoNvlsStaged, (int)DevColl::allreduce);
  for (uint64_t c = 0; c < G; ++c) {
    const int par = (int)((P.seq + c) & 1);
    char* mystage = ws.stage[rank] + (size_t)par * half;
    char* mc = ws.mc_stage + (size_t)par * half;
    const size_t base = c * full_e, len = clamp_len(P.count, base, full_e);
    size_t lo, hi;
    split_range(len, blockIdx.x, gridDim.x, 16 / sizeof(T), lo, hi);
    if (hi > lo) cta_copy(mystage + lo * sizeof(T), (const char*)(send + base + lo), (hi - lo) * sizeof(T), false);

    const uint64_t e = make_epoch(P.seq, c + 1);
    arrive_and_post(ws, rank, FlagLayout::off_A, 0, gridDim.x, e, c == 0, (int)(P.seq & 1), G, my_proto);
    if (!wait_all(ws, rank, FlagLayout::off_A, 0, e, P.timeout_ns)) return;
    if (c == 0 && !protocols_agree(ws, rank, P.seq, my_proto)) return;

    const size_t nvec = (len * sizeof(T) + 15) >> 4;  // the tail vector may include stale bytes: harmless
    size_t s_lo, s_hi;
    split_range(nvec, (unsigned)rank, (unsigned)p, 1, s_lo, s_hi);
    reduce_vectors<T, OP>(mc, mc, s_lo, s_hi, scale, blockIdx.x, gridDim.x);
    __threadfence_system();
    arrive_and_post(ws, rank, FlagLayout::off_B, 1, gridDim.x, e, false, 0, 0);
    if (!wait_all(ws, rank, FlagLayout::off_B, 1, e, P.timeout_ns)) return;

    if (hi > lo) cta_copy((char*)(recv + base + lo), mystage + lo * sizeof(T), (hi - lo) * sizeof(T), true);
  }
  if (G > 1) {
    const uint64_t e = make_epoch(P.seq, 1);
    arrive_and_post(ws, rank, FlagLayout::off_C, 2, gridDim.x, e, false, 0, 0);
    (void)wait_all(ws, rank, FlagLayout::off_C, 2, e, P.timeout_ns);
  }
}

/**
 * Staged NVLS allreduce for large private buffers, software-pipelined over chunks by
 * three groups of CTAs that run concurrently:
 *   IN   copies chunk c of the user's input into the multicast-bound staging half (HBM),
 *   RED  switch-reduces this rank's slice of chunk c in place (NVLink),
 *   OUT  copies the finished chunk to the user's output (HBM),
 * so that the copies of neighbouring chunks hide behind the NVLink phase.  The chunks travel through a
 * ring of D slots laid over both staging halves (D = 2 * half / chunk, at most kRingDepth), so IN may run
 * D-1 chunks ahead of OUT and a late copy never stalls the switch phase.  Flags:
 * A(c) "my copy-in of chunk c is done" (to everyone), B(c) "my slice of chunk c is
 * reduced and replicated" (to everyone), C(c) "I copied chunk c out" (to everyone;
 * IN only looks at its own, the closing wait looks at all).
 */
template <typename T, NvOp OP>
__global__ void __launch_bounds__(512) nvls_allreduce_pipelined_kernel(const __grid_constant__ NvlsParams P) {
  const Workspace& ws = P.ws;
  const int p = ws.p, rank = P.rank;
  if (poisoned(ws, rank)) return;
  const float scale = (float)P.scale;
  const size_t chunk_e = P.chunk_elems;
  const size_t chunk_b = chunk_e * sizeof(T);   // a multiple of 4096; ring slot c % D starts at (c % D) * chunk_b
  const int D = P.ring_depth;                   // slots in the staging area (both halves, contiguous)
  const uint64_t G = P.chunks;
  const T* send = (const T*)P.send;
  T* recv = (T*)P.recv;
  const unsigned n = gridDim.x;
  unsigned n_red = n / 4 < 4 ? 4 : n / 4;
  if (n_red > n - 2) n_red = n - 2;
  const unsigned n_in = (n - n_red) / 2, n_out = n - n_red - n_in;
  const unsigned b = blockIdx.x;
  const uint64_t my_proto = proto_word(kProtoNvlsStaged, (int)DevColl::allreduce, 1);

  if (b < n_in) {
    for (uint64_t c = 0; c < G; ++c) {
      if (c >= (uint64_t)D) {  // the slot is free once my own OUT group copied chunk c-D out (which follows every rank's RED of it)
        __shared__ int s_ok;
        if (threadIdx.x == 0) {
          uint64_t seen = 0;
          s_ok = wait_flag(flag_slot(ws.flags[rank], FlagLayout::off_C, rank), make_epoch(P.seq, c - D + 1), P.timeout_ns, &seen);
          if (!s_ok) report_timeout(ws, rank, rank, 2, make_epoch(P.seq, c - D + 1), seen);
        }
        __syncthreads();
        if (!s_ok) return;
      }
      char* mystage = ws.stage[rank] + (size_t)(c % D) * chunk_b;
      const size_t base = c * chunk_e, len = clamp_len(P.count, base, chunk_e);
      size_t lo, hi;
      split_range(len, b, n_in, 16 / sizeof(T), lo, hi);
      if (hi > lo) cta_copy(mystage + lo * sizeof(T), (const char*)(send + base + lo), (hi - lo) * sizeof(T), false);
      arrive_and_post_ring(ws, rank, FlagLayout::off_A, 0, c, D, n_in, make_epoch(P.seq, c + 1), c == 0, (int)(P.seq & 1), G, my_proto);
    }
  } else if (b < n_in + n_red) {
    // Two sub-groups take the even and the odd chunks: while one of them waits for its stores to be
    // acknowledged and posts its flags, the other one keeps the links busy.  Each parity has its own B word
    // (word 0 / word 1 of the flag's sector), so that every word only ever grows.
    const unsigned rb = b - n_in;
    const unsigned nsub = n_red >= 8 && D >= 4 ? 2 : 1;
    const unsigned sub = rb % nsub, part = rb / nsub;
    const unsigned ns = n_red / nsub + (sub < n_red % nsub ? 1 : 0);
    for (uint64_t c = sub; c < G; c += nsub) {
      if (!wait_all(ws, rank, FlagLayout::off_A, 0, make_epoch(P.seq, c + 1), P.timeout_ns)) return;
      if (c == sub && !protocols_agree(ws, rank, P.seq, my_proto)) return;
      char* mc = ws.mc_stage + (size_t)(c % D) * chunk_b;
      const size_t base = c * chunk_e, len = clamp_len(P.count, base, chunk_e);
      const size_t nvec = (len * sizeof(T) + 15) >> 4;
      size_t s_lo, s_hi;
      split_range(nvec, (unsigned)rank, (unsigned)p, 1, s_lo, s_hi);
      reduce_vectors<T, OP>(mc, mc, s_lo, s_hi, scale, part, ns);
      __threadfence_system();
      arrive_and_post_ring(ws, rank, FlagLayout::off_B, 1, c, D, ns, make_epoch(P.seq, c + 1), false, 0, 0, 0, (int)(c & 1));
    }
  } else {
    for (uint64_t c = 0; c < G; ++c) {
      if (!wait_all(ws, rank, FlagLayout::off_B, 1, make_epoch(P.seq, c + 1), P.timeout_ns, (int)(c & 1))) return;
      char* mystage = ws.stage[rank] + (size_t)(c % D) * chunk_b;
      const size_t base = c * chunk_e, len = clamp_len(P.count, base, chunk_e);
      size_t lo, hi;
      split_range(len, b - n_in - n_red, n_out, 16 / sizeof(T), lo, hi);
      if (hi > lo) cta_copy((char*)(recv + base + lo), mystage + lo * sizeof(T), (hi - lo) * sizeof(T), true);
      arrive_and_post_ring(ws, rank, FlagLayout::off_C, 2, c, D, n_out, make_epoch(P.seq, c + 1), false, 0, 0);
    }
  }
  // Closing barrier: every rank has copied its last chunk out; the whole staging area is free for the next launch.
  (void)wait_all(ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, G), P.timeout_ns);
}

/**
 * Staged NVLS reduce_scatter for large private buffers: the switch reduces, two groups of CTAs pipeline.
 *   IN   copies chunk c of all p slices of the user's input into the multicast-bound staging half,
 *        slice d at slot d (HBM traffic only), and posts A(c) to everyone;
 *   RED  waits for everyone's A(c), pulls this rank's slot through multimem.ld_reduce - one reduced stream
 *        arrives instead of p-1 pushed ones, and nothing is read back from staging - applies the scale,
 *        writes the user's output and posts C(c) to everyone.
 * A staging half is reused every second chunk: IN waits for everyone's C(c-2) first, because every rank's RED
 * group reads every rank's staging.  `count` is the length of one slice, `chunk_elems` the part of a slice
 * that travels per chunk.  (Role of ncclReduceScatter's NVLS kernels behind the reference,
 * include/aluminum/nccl_impl.hpp:1306.)
 */
template <typename T, NvOp OP>
__global__ void __launch_bounds__(512) nvls_reduce_scatter_kernel(const __grid_constant__ NvlsParams P) {
  constexpr int VEC = 16 / (int)sizeof(T);
  const Workspace& ws = P.ws;
  const int p = ws.p, rank = P.rank;
  if (poisoned(ws, rank)) return;
  const float scale = (float)P.scale;
  const size_t half = ws.half_bytes;
  const size_t cap_b = (half / (size_t)p) / 256 * 256;  // one slot per slice
  const size_t chunk_e = P.chunk_elems;
  const uint64_t G = P.chunks;
  const T* send = (const T*)P.send;
  T* recv = (T*)P.recv;
  const unsigned n = gridDim.x, b = blockIdx.x;
  const unsigned n_red = n / 2 < 1 ? 1 : n / 2, n_in = n - n_red;
  const uint64_t my_proto = proto_word(kProtoNvlsStaged, (int)DevColl::reduce_scatter, 1);
  // Ranks that took the window path wait for this flag before they touch anything: tell them what runs here.
  if (b == 0) post_entered(ws, rank, P.seq, my_proto, 0, 0);

  if (b < n_in) {
    for (uint64_t c = 0; c < G; ++c) {
      if (c >= 2 && !wait_all(ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, c - 1), P.timeout_ns)) return;
      char* mystage = ws.stage[rank] + (size_t)((P.seq + c) & 1) * half;
      const size_t base = c * chunk_e, len = clamp_len(P.count, base, chunk_e);
      size_t lo, hi;
      split_range(len, b, n_in, (size_t)VEC, lo, hi);
      if (hi > lo)
        for (int i = 0; i < p; ++i) {
          const int d = (rank + i) % p;
          cta_copy(mystage + (size_t)d * cap_b + lo * sizeof(T), (const char*)(send + (size_t)d * P.count + base + lo),
                   (hi - lo) * sizeof(T), false);
        }
      arrive_and_post(ws, rank, FlagLayout::off_A, 0, n_in, make_epoch(P.seq, c + 1), c == 0, (int)(P.seq & 1), G, my_proto);
    }
  } else {
    const unsigned part = b - n_in;
    for (uint64_t c = 0; c < G; ++c) {
      if (!wait_all(ws, rank, FlagLayout::off_A, 0, make_epoch(P.seq, c + 1), P.timeout_ns)) return;
      if (c == 0 && !protocols_agree(ws, rank, P.seq, my_proto)) return;
      const char* mc = ws.mc_stage + (size_t)((P.seq + c) & 1) * half + (size_t)rank * cap_b;
      const size_t base = c * chunk_e, len = clamp_len(P.count, base, chunk_e);
      const size_t nvec = (len + VEC - 1) / VEC;  // the tail vector reads stale staging bytes; store_group drops them
      T* out = recv + base;
      constexpr int U = 4;
      const size_t stride = (size_t)blockDim.x * n_red;
      size_t v = (size_t)part * blockDim.x + threadIdx.x;
      for (; v + (U - 1) * stride < nvec; v += U * stride) {
        uint4 a[U];
#pragma unroll
        for (int u = 0; u < U; ++u) a[u] = MM<T, OP>::ld(mc + ((v + u * stride) << 4));
#pragma unroll
        for (int u = 0; u < U; ++u) {
          if (scale != 1.f) a[u] = scale_pack<T>(a[u], scale);
          store_group(out, (v + u * stride) * VEC, len, a[u]);
        }
      }
      for (; v < nvec; v += stride) {
        uint4 a = MM<T, OP>::ld(mc + (v << 4));
        if (scale != 1.f) a = scale_pack<T>(a, scale);
        store_group(out, v * VEC, len, a);
      }
      arrive_and_post(ws, rank, FlagLayout::off_C, 2, n_red, make_epoch(P.seq, c + 1), false, 0, 0);
    }
  }
  // Closing barrier: every rank has pulled its last chunk, both halves are free for the next launch.
  (void)wait_all(ws, rank, FlagLayout::off_C, 2, make_epoch(P.seq, G), P.timeout_ns);
}

template <typename T, NvOp OP>
void launch(const NvlsParams& P, int ctas, int threads, cudaStream_t s) {
  if (P.chunk_elems && !P.mc_in && ctas >= 8) {
    nvls_allreduce_pipelined_kernel<T, OP><<<ctas, threads, 0, s>>>(P);
    AL_CHECK_CUDA(cudaGetLastError());
    return;
  }
  nvls_allreduce_kernel<T, OP><<<ctas, threads, 0, s>>>(P);
  AL_CHECK_CUDA(cudaGetLastError());
}

}  // namespace

bool nvls_allreduce_supported(DType dt, ReductionOperator op) {
  const bool add = op == ReductionOperator::sum || op == ReductionOperator::avg;
  if (dt == DType::f32) return add;
  if (dt == DType::bf16 || dt == DType::f16)
    return add || op == ReductionOperator::min || op == ReductionOperator::max;
  return false;
}

void launch_nvls_allreduce(const NvlsParams& P, DType dt, ReductionOperator op, int ctas, int threads,
                           cudaStream_t s) {
  if (!nvls_allreduce_supported(dt, op)) throw_al_exception("NVLS allreduce does not support this type/operator");
  const bool add = op == ReductionOperator::sum || op == ReductionOperator::avg;
  if (dt == DType::f32) return launch<float, NvOp::add>(P, ctas, threads, s);
  if (dt == DType::bf16) {
    if (add) return launch<__nv_bfloat16, NvOp::add>(P, ctas, threads, s);
    if (op == ReductionOperator::min) return launch<__nv_bfloat16, NvOp::min>(P, ctas, threads, s);
    return launch<__nv_bfloat16, NvOp::max>(P, ctas, threads, s);
  }
  if (add) return launch<__half, NvOp::add>(P, ctas, threads, s);
  if (op == ReductionOperator::min) return launch<__half, NvOp::min>(P, ctas, threads, s);
  return launch<__half, NvOp::max>(P, ctas, threads, s);
}

template <typename T, NvOp OP>
static void launch_rs(const NvlsParams& P, int ctas, int threads, cudaStream_t s) {
  nvls_reduce_scatter_kernel<T, OP><<<ctas, threads, 0, s>>>(P);
  AL_CHECK_CUDA(cudaGetLastError());
}

void launch_nvls_reduce_scatter(const NvlsParams& P, DType dt, ReductionOperator op, int ctas, int threads,
                                cudaStream_t s) {
  if (!nvls_allreduce_supported(dt, op)) throw_al_exception("NVLS reduce_scatter does not support this type/operator");
  if (ctas < 2) ctas = 2;
  const bool add = op == ReductionOperator::sum || op == ReductionOperator::avg;
  if (dt == DType::f32) return launch_rs<float, NvOp::add>(P, ctas, threads, s);
  if (dt == DType::bf16) {
    if (add) return launch_rs<__nv_bfloat16, NvOp::add>(P, ctas, threads, s);
    if (op == ReductionOperator::min) return launch_rs<__nv_bfloat16, NvOp::min>(P, ctas, threads, s);
    return launch_rs<__nv_bfloat16, NvOp::max>(P, ctas, threads, s);
  }
  if (add) return launch_rs<__half, NvOp::add>(P, ctas, threads, s);
  if (op == ReductionOperator::min) return launch_rs<__half, NvOp::min>(P, ctas, threads, s);
  return launch_rs<__half, NvOp::max>(P, ctas, threads, s);
}

}  // namespace device
}  // namespace internal
}  // namespace Al
