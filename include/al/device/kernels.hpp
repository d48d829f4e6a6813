/**
 * @file kernels.hpp
 * Host-callable launchers of every sm_100a kernel in the library.  The
 * communicator layer (al/device/communicator.hpp) decides algorithm, grid
 * and arguments; these functions only launch.
 *
 * The reference contains no data-path kernels at all - each operation is one
 * NCCL call (include/aluminum/nccl_impl.hpp:944-1399) or a cudaMemcpyPeerAsync
 * (include/aluminum/mpi_cuda/rma_ipc.hpp:298-299); these kernels are what
 * replaces those calls.
 */
#pragma once
#include <cuda_runtime.h>

#include "al/base.hpp"
#include "al/device/params.hpp"

namespace Al {
namespace internal {
namespace device {

// ---- generic staged collectives (kernels/coll_*.cu) --------------------------
/**
 * Launch the collective kernel for element types (in, wire, out).  For pure
 * data movement pass DType::u8 three times and counts in bytes.
 * @param ctas        grid.x (same on every rank of the communicator)
 * @param local_ranks grid.y; > 1 launches cooperatively (single-GPU emulation)
 */
void launch_collective(const CollParams& P, DType in, DType wire, DType out, int ctas, int threads,
                       int local_ranks, cudaStream_t stream);
/** True when (in, wire, out, op) has a compiled kernel. */
bool collective_supported(DType in, DType wire, DType out, ReductionOperator op);

// ---- bulk-copy pipeline (kernels/bulk_pipeline.cu) ------------------------------
/**
 * Large uniform allgather / alltoall (dt = u8, counts in bytes) and sum
 * reduce_scatter (f32 / f16 / bf16) with the copy engine (cp.async.bulk) moving
 * the data; protocol-compatible with the pipelined schedule of the generic
 * kernel.  Requirements checked by the caller: P.pipelined, every send / recv
 * pointer 16-byte aligned, the per-rank slice a multiple of 16 bytes.
 */
bool bulk_pipeline_supported(DevColl kind, DType dt, ReductionOperator op);
void launch_bulk_pipeline(const CollParams& P, DType dt, int ctas, int threads, int local_ranks, cudaStream_t stream);

// ---- low-latency kernel (kernels/ll.cu) ------------------------------------------------------
/**
 * Small uniform allreduce / reduce_scatter (same in, wire and out type) and allgather / alltoall (dt = u8,
 * counts in bytes): at most kLLPayloadBytes from one rank to another, count > 0.
 */
bool ll_supported(DevColl kind, DType dt, ReductionOperator op);
void launch_ll(const LLParams& P, DType dt, int ctas, int threads, int local_ranks, cudaStream_t stream);

// ---- row exchange (kernels/rows.cu) --------------------------------------------------------------
/** Alltoall(v) of strided / indexed rows through the staging area (see RowsParams). */
void launch_rows(const RowsParams& P, int ctas, int threads, int local_ranks, cudaStream_t stream);

// ---- window kernels (kernels/window.cu) ----------------------------------------------
/**
 * Uniform reduce_scatter (f32 / f16 / bf16; sum, avg, min, max) and allgather / alltoall / bcast (counts in
 * bytes) straight on registered buffers: no staging.  P.windows must point to the communicator's window
 * table in device memory and the descriptors of the registered side must be filled in (see WinParams).
 */
bool window_supported(DevColl kind, DType dt, ReductionOperator op);
void launch_window(const WinParams& P, DType dt, ReductionOperator op, int ctas, int threads, int local_ranks,
                   cudaStream_t stream);

// ---- NVLS allreduce (kernels/nvls.cu) ------------------------------------------
struct NvlsParams {
  Workspace ws;
  const void* send;     ///< staged flavour: private input
  void* recv;           ///< staged flavour: private output
  const char* mc_in;    ///< zero-copy flavour: multicast alias of the symmetric input (nullptr = staged)
  char* mc_out;         ///< zero-copy flavour: multicast alias of the symmetric output
  size_t count;
  size_t chunk_elems;   ///< non-zero: pipelined staged flavour with chunks of this many elements
  int ring_depth;       ///< pipelined allreduce: chunks in flight (slots of chunk_elems laid over both staging halves)
  uint64_t chunks;
  uint64_t seq;
  uint64_t timeout_ns;
  double scale;
  int rank;
};
bool nvls_allreduce_supported(DType dt, ReductionOperator op);
void launch_nvls_allreduce(const NvlsParams& P, DType dt, ReductionOperator op, int ctas, int threads,
                           cudaStream_t stream);
/** Staged NVLS reduce_scatter of private buffers (same types / operators): `count` = elements per slice,
 *  `chunk_elems` = elements of a slice per chunk (at most a p-th of a staging half), `chunks` accordingly. */
void launch_nvls_reduce_scatter(const NvlsParams& P, DType dt, ReductionOperator op, int ctas, int threads,
                                cudaStream_t stream);

// ---- point-to-point mailbox transfers (kernels/p2p.cu) ----------------------------
void launch_p2p(const P2PParams& P, int threads, int local_ranks_cooperative, cudaStream_t stream);

// ---- RMA and halo exchange (kernels/rma_halo.cu) ------------------------------------
/** Contiguous put: copy `bytes` from local `src` to the peer-mapped `dst` with SM stores. */
void launch_put(void* dst_peer, const void* src, size_t bytes, int ctas, cudaStream_t stream);
/** Store `value` (release, system scope) into a peer-mapped 64-bit word. */
void launch_signal(uint64_t* peer_word, uint64_t value, cudaStream_t stream);
/** Wait (bounded) until a local 64-bit word reaches `value`; on time-out fills `status`. */
void launch_wait_word(const uint64_t* word, uint64_t value, uint64_t timeout_ns, Workspace ws, int rank,
                      int peer, cudaStream_t stream);

/**
 * Fused halo exchange for a tensor laid out (N, C, D, H, W), contiguous, split
 * along D.  One launch packs the `depth` boundary planes next to each
 * neighbour straight out of the interior, stores them into the neighbour's
 * halo planes through its peer-mapped tensor, and signals; a second phase in
 * the same kernel waits for both neighbours' signals.  No pack buffer and no
 * separate unpack kernel exist: the peer store lands in its final place.
 */
struct HaloParams {
  Workspace ws;
  float* tensor[kMaxRanks]; ///< every rank's tensor (incl. halo planes) as mapped here: (NC, D_local + 2*depth, H*W);
                            ///< only the executing rank(s) and their neighbours need valid entries
  int lo[kMaxRanks];        ///< lower neighbour of each rank, -1 at the boundary
  int hi[kMaxRanks];        ///< upper neighbour, -1 at the boundary
  size_t nc;                ///< N*C
  size_t d_local;           ///< interior planes per rank
  size_t plane;             ///< H*W elements
  size_t depth;             ///< halo depth in planes
  uint64_t epoch;           ///< value signalled to / expected from the neighbours
  uint64_t timeout_ns;
  int rank0;                ///< block (x, y) works for rank rank0 + y
};
/** local_ranks > 1 launches cooperatively (single-GPU emulation of all ranks). */
void launch_halo_exchange(const HaloParams& P, int ctas, int threads, int local_ranks, cudaStream_t stream);
/** Stand-alone pack / unpack of boundary planes (for the unfused comparison path). */
void launch_halo_pack(float* packed, const float* tensor, size_t nc, size_t d_total, size_t plane,
                      size_t d_first, size_t depth, cudaStream_t stream);
void launch_halo_unpack(float* tensor, const float* packed, size_t nc, size_t d_total, size_t plane,
                        size_t d_first, size_t depth, cudaStream_t stream);

// ---- element-wise kernels (kernels/elementwise.cu) -----------------------------------
/** out[i] = (Tout)(in[i] * scale); in and out may alias when the types match. */
void launch_scale_cast(void* out, DType out_dt, const void* in, DType in_dt, size_t n, double scale,
                       cudaStream_t stream);
/**
 * Fused momentum-SGD over a flat fp32 parameter buffer:
 *   g = grad*grad_scale + wd*p;  m = mu*m + g (m = g on the first step);  p -= lr*m
 * and optionally zero the gradient afterwards.
 */
void launch_sgd_momentum(float* param, float* momentum, float* grad, size_t n, float lr, float mu,
                         float weight_decay, float grad_scale, int first_step, int zero_grad,
                         cudaStream_t stream);
/** Fill with a 32-bit pattern (used by tests and benchmarks to flush L2). */
void launch_fill_u32(uint32_t* out, size_t n, uint32_t value, cudaStream_t stream);

}  // namespace device
}  // namespace internal
}  // namespace Al
