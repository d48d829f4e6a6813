// RMA building blocks (put / signal / bounded wait) and the fused halo exchange.
//
// The reference's put is a cudaMemcpyPeerAsync on the communicator's stream and
// its notify/wait/sync are host handshakes run by the progress engine
// (include/aluminum/mpi_cuda/rma_ipc.hpp:40-148,287-301).  Here a put is a
// grid of SM stores into the peer-mapped buffer and notify/wait are a release
// store to / a bounded acquire poll of a 64-bit word in symmetric memory, all
// ordered on the communicator's stream with no host involvement.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

__global__ void __launch_bounds__(512) put_kernel(char* dst, const char* src, size_t bytes) {
  size_t lo, hi;
  split_range(bytes, blockIdx.x, gridDim.x, 16, lo, hi);
  if (hi > lo) cta_copy(dst + lo, src + lo, hi - lo, false);
}

__global__ void signal_kernel(uint64_t* word, uint64_t value) {
  __threadfence_system();
  st_release_sys(word, value);
}

__global__ void wait_word_kernel(const uint64_t* word, uint64_t value, uint64_t timeout_ns, Workspace ws,
                                 int rank, int peer) {
  if (poisoned(ws, rank)) return;
  uint64_t seen = 0;
  if (!wait_flag(word, value, timeout_ns, &seen)) report_timeout(ws, rank, peer, 5, value, seen);
}

/**
 * Copy, for every channel, `depth` planes starting at plane `src_first` of the
 * local tensor to planes starting at `dst_first` of `dst` (same shape).  The
 * work (nc * depth * plane floats) is split evenly over `nparts` CTAs.
 */
__device__ __forceinline__ void copy_planes(float* dst, const float* src, size_t nc, size_t d_total, size_t plane,
                                            size_t src_first, size_t dst_first, size_t depth, unsigned part,
                                            unsigned nparts) {
  const size_t seg = depth * plane;  // contiguous floats per channel
  const size_t total = nc * seg;
  size_t lo, hi;
  split_range(total, part, nparts, 4, lo, hi);
  while (lo < hi) {
    const size_t c = lo / seg, within = lo - c * seg;
    size_t len = seg - within;
    if (len > hi - lo) len = hi - lo;
    const float* s = src + (c * d_total + src_first) * plane + within;
    float* d = dst + (c * d_total + dst_first) * plane + within;
    cta_copy((char*)d, (const char*)s, len * sizeof(float), false);
    lo += len;
  }
}

__global__ void __launch_bounds__(512) halo_exchange_kernel(const __grid_constant__ HaloParams P) {
  const Workspace& ws = P.ws;
  const int rank = P.rank0 + (int)blockIdx.y;
  if (poisoned(ws, rank)) return;
  uint64_t* mine = ws.flags[rank];
  const size_t d_total = P.d_local + 2 * P.depth;
  const int lo_rank = P.lo[rank], hi_rank = P.hi[rank];
  const bool has_lo = lo_rank >= 0, has_hi = hi_rank >= 0;
  const float* local = P.tensor[rank];
  float* peer_lo = has_lo ? P.tensor[lo_rank] : nullptr;
  float* peer_hi = has_hi ? P.tensor[hi_rank] : nullptr;

  // 1. Tell both neighbours that my halo planes may be overwritten (this
  //    kernel is stream-ordered after whatever consumed them last).
  if (blockIdx.x == 0 && threadIdx.x == 0) {
    if (has_lo) st_release_sys(flag_slot(ws.flags[lo_rank], FlagLayout::off_halo, 1), P.epoch);  // I am its "hi"
    if (has_hi) st_release_sys(flag_slot(ws.flags[hi_rank], FlagLayout::off_halo, 0), P.epoch);  // I am its "lo"
  }
  // 2. Wait until the neighbours said the same.
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < 2) {
    const bool need = threadIdx.x == 0 ? has_lo : has_hi;
    if (need) {
      uint64_t seen = 0;
      if (!wait_flag(flag_slot(mine, FlagLayout::off_halo, threadIdx.x), P.epoch, P.timeout_ns, &seen)) {
        report_timeout(ws, rank, threadIdx.x == 0 ? lo_rank : hi_rank, 5, P.epoch, seen);
        s_ok = 0;
      }
    }
  }
  __syncthreads();
  if (!s_ok) return;

  // 3. Peer stores: the first half of the grid serves the lower neighbour, the
  //    second half the upper one (all CTAs serve one side at a boundary rank).
  const unsigned n = gridDim.x;
  if (has_lo && has_hi && n >= 2) {
    const unsigned h = n / 2;
    if (blockIdx.x < h)
      copy_planes(peer_lo, local, P.nc, d_total, P.plane, P.depth, P.depth + P.d_local, P.depth, blockIdx.x, h);
    else
      copy_planes(peer_hi, local, P.nc, d_total, P.plane, P.d_local, 0, P.depth, blockIdx.x - h, n - h);
  } else {
    if (has_lo) copy_planes(peer_lo, local, P.nc, d_total, P.plane, P.depth, P.depth + P.d_local, P.depth, blockIdx.x, n);
    if (has_hi) copy_planes(peer_hi, local, P.nc, d_total, P.plane, P.d_local, 0, P.depth, blockIdx.x, n);
  }

  // 4. The last CTA to finish publishes "data landed" to both neighbours.
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    int last = 1;
    if (n > 1) last = atomicInc((unsigned*)flag_slot(mine, FlagLayout::off_arrive, 3), n - 1) == n - 1;
    if (last) {
      __threadfence_system();
      if (has_lo) st_release_sys(flag_slot(ws.flags[lo_rank], FlagLayout::off_halo, 3), P.epoch);
      if (has_hi) st_release_sys(flag_slot(ws.flags[hi_rank], FlagLayout::off_halo, 2), P.epoch);
    }
  }
  __syncthreads();

  // 5. Wait for the neighbours' data so that the kernel's completion means
  //    "my halos are filled".
  if (threadIdx.x < 2) {
    const bool need = threadIdx.x == 0 ? has_lo : has_hi;
    if (need) {
      uint64_t seen = 0;
      if (!wait_flag(flag_slot(mine, FlagLayout::off_halo, 2 + threadIdx.x), P.epoch, P.timeout_ns, &seen))
        report_timeout(ws, rank, threadIdx.x == 0 ? lo_rank : hi_rank, 5, P.epoch, seen);
    }
  }
}

__global__ void __launch_bounds__(512) halo_pack_kernel(float* packed, const float* tensor, size_t nc, size_t d_total,
                                                        size_t plane, size_t d_first, size_t depth, int unpack) {
  const size_t seg = depth * plane, total = nc * seg;
  size_t lo, hi;
  split_range(total, blockIdx.x, gridDim.x, 4, lo, hi);
  while (lo < hi) {
    const size_t c = lo / seg, within = lo - c * seg;
    size_t len = seg - within;
    if (len > hi - lo) len = hi - lo;
    const float* t = tensor + (c * d_total + d_first) * plane + within;
    float* pk = packed + lo;
    if (unpack) cta_copy((char*)t, (const char*)pk, len * sizeof(float), false);
    else cta_copy((char*)pk, (const char*)t, len * sizeof(float), false);
    lo += len;
  }
}

}  // namespace

void launch_put(void* dst_peer, const void* src, size_t bytes, int ctas, cudaStream_t stream) {
  if (bytes == 0) return;
  put_kernel<<<ctas, 512, 0, stream>>>((char*)dst_peer, (const char*)src, bytes);
  AL_CHECK_CUDA(cudaGetLastError());
}

void launch_signal(uint64_t* peer_word, uint64_t value, cudaStream_t stream) {
  signal_kernel<<<1, 1, 0, stream>>>(peer_word, value);
  AL_CHECK_CUDA(cudaGetLastError());
}

void launch_wait_word(const uint64_t* word, uint64_t value, uint64_t timeout_ns, Workspace ws, int rank, int peer,
                      cudaStream_t stream) {
  wait_word_kernel<<<1, 1, 0, stream>>>(word, value, timeout_ns, ws, rank, peer);
  AL_CHECK_CUDA(cudaGetLastError());
}

void launch_halo_exchange(const HaloParams& P, int ctas, int threads, int local_ranks, cudaStream_t stream) {
  dim3 grid((unsigned)ctas, (unsigned)local_ranks);
  void* args[] = {(void*)&P};
  if (local_ranks > 1)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)halo_exchange_kernel, grid, dim3((unsigned)threads), args, 0, stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)halo_exchange_kernel, grid, dim3((unsigned)threads), args, 0, stream));
}

void launch_halo_pack(float* packed, const float* tensor, size_t nc, size_t d_total, size_t plane, size_t d_first,
                      size_t depth, cudaStream_t stream) {
  halo_pack_kernel<<<148, 512, 0, stream>>>(packed, tensor, nc, d_total, plane, d_first, depth, 0);
  AL_CHECK_CUDA(cudaGetLastError());
}

void launch_halo_unpack(float* tensor, const float* packed, size_t nc, size_t d_total, size_t plane, size_t d_first,
                        size_t depth, cudaStream_t stream) {
  halo_pack_kernel<<<148, 512, 0, stream>>>(const_cast<float*>(packed), tensor, nc, d_total, plane, d_first, depth, 1);
  AL_CHECK_CUDA(cudaGetLastError());
}

}  // namespace device
}  // namespace internal
}  // namespace Al
