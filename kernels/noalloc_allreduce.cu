// Allocation-free single-GPU allreduce (see al/noalloc.h for who needs it and the rules).
// The kernel is the library's generic collective kernel, launched cooperatively over p
// emulated ranks; only the origin of its workspace differs: a static device array
// instead of a communicator's allocation.
#include "al/noalloc.h"

#include <mutex>
#include <string>

#include "coll_launch.cuh"

using namespace Al::internal::device;

namespace {

constexpr size_t kSlotBytes = 32768;                                  // AL_NOALLOC_MAX_COUNT floats
constexpr size_t kHalfBytes = AL_NOALLOC_MAX_RANKS * kSlotBytes;      // one slot per source rank
constexpr size_t kRankBytes = FlagLayout::bytes + 2 * kHalfBytes;
static_assert(FlagLayout::bytes == 4096, "scratch size in the header assumes a 4 KiB flag area");
static_assert(AL_NOALLOC_SCRATCH_BYTES == AL_NOALLOC_MAX_RANKS * kRankBytes, "header constant out of date");
static_assert(AL_NOALLOC_MAX_COUNT * sizeof(float) == kSlotBytes, "slot must hold the largest vector");

// The scratch: flags + two staging halves for each of up to 8 emulated ranks.  Zero-initialised
// when the module is loaded; afterwards it keeps whatever the last call wrote.
static __device__ __align__(256) unsigned char g_noalloc_scratch[AL_NOALLOC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
struct PerDevice {
  unsigned char* base = nullptr;   // device address of g_noalloc_scratch on this device
  uint64_t seq = 0;                // epochs continue across calls, so flags never need resetting
};
PerDevice g_dev[kMaxDevices];
std::mutex g_mu;
thread_local std::string g_err;

int fail(const std::string& msg) {
  g_err = msg;
  return 1;
}

}  // namespace

extern "C" const char* al_noalloc_last_error(void) { return g_err.c_str(); }

extern "C" int al_noalloc_allreduce_f32(const float* const* inputs, float* const* outputs, int p, size_t count,
                                        void* stream) {
  if (p < 1 || p > AL_NOALLOC_MAX_RANKS)
    return fail("al_noalloc_allreduce_f32: p must be between 1 and " + std::to_string(AL_NOALLOC_MAX_RANKS));
  if (count > AL_NOALLOC_MAX_COUNT)
    return fail("al_noalloc_allreduce_f32: count " + std::to_string(count) + " exceeds the built-in scratch (" +
                std::to_string(AL_NOALLOC_MAX_COUNT) + " fp32 elements per rank)");
  if (!inputs || !outputs) return fail("al_noalloc_allreduce_f32: null argument");
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail("al_noalloc_allreduce_f32: device index out of range");

  std::lock_guard<std::mutex> lock(g_mu);
  PerDevice& D = g_dev[dev];
  if (!D.base) {
    // Set-up, once per device, with that device current: in host code the array's name is only a
    // stand-in; the address a kernel can use has to be asked for.
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) return fail(std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
    D.base = (unsigned char*)ptr;
  }

  CollParams P{};
  P.ws.p = p;
  P.ws.half_bytes = kHalfBytes;
  P.ws.mbox_slot_bytes = 0;
  P.ws.mc_stage = nullptr;
  P.ws.status = nullptr;  // no pinned status record: a timed-out wait only marks the flag area (al_noalloc_status reads it)
  for (int r = 0; r < p; ++r) {
    unsigned char* rb = D.base + (size_t)r * kRankBytes;
    P.ws.flags[r] = (uint64_t*)rb;
    P.ws.stage[r] = (char*)rb + FlagLayout::bytes;
    P.ws.mbox[r] = nullptr;
    if (count && (!inputs[r] || !outputs[r])) return fail("al_noalloc_allreduce_f32: null buffer for a rank");
    P.send[r] = inputs[r];
    P.recv[r] = outputs[r];
    for (int i = 0; i < p; ++i) {
      P.tab[r].send_counts[i] = P.tab[r].recv_counts[i] = count;
      P.tab[r].send_displs[i] = P.tab[r].recv_displs[i] = (size_t)i * count;
    }
    P.local_chunks[r] = 1;
  }
  P.seq = ++D.seq;
  P.timeout_ns = 2000000000ull;
  P.count = count;
  P.scale = 1.0;
  P.int_div = 1;
  P.kind = (int)DevColl::allreduce;
  P.op = (int)Al::ReductionOperator::sum;
  P.root = 0;
  P.rank0 = 0;
  P.two_phase = 0;
  P.pipelined = 0;
  P.slot_elems = 0;

  RedSum red;
  void* args[] = {(void*)&P, (void*)&red};
  auto k = coll_kernel<float, float, float, RedSum>;
  const dim3 grid(1, (unsigned)p, 1), block(256, 1, 1);
  if (p > 1) e = cudaLaunchCooperativeKernel((const void*)k, grid, block, args, 0, (cudaStream_t)stream);
  else e = cudaLaunchKernel((const void*)k, grid, block, args, 0, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("launch failed: ") + cudaGetErrorString(e));
  return 0;
}

// ---------------------------------------------------------------------------------------------
// status and recovery
// ---------------------------------------------------------------------------------------------
namespace {
/** Device address of the scratch on the current device (looked up on first use), or nullptr + error. */
PerDevice* current_device_state() {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { fail(std::string("cudaGetDevice: ") + cudaGetErrorString(e)); return nullptr; }
  if (dev < 0 || dev >= kMaxDevices) { fail("al_noalloc: device index out of range"); return nullptr; }
  PerDevice& D = g_dev[dev];
  if (!D.base) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || !ptr) { fail(std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e)); return nullptr; }
    D.base = (unsigned char*)ptr;
  }
  return &D;
}
}  // namespace

extern "C" int al_noalloc_status(int* code) {
  if (!code) return fail("al_noalloc_status: null argument");
  std::lock_guard<std::mutex> lock(g_mu);
  PerDevice* D = current_device_state();
  if (!D) return 1;
  *code = 0;
  for (int r = 0; r < AL_NOALLOC_MAX_RANKS; ++r) {
    unsigned long long word = 0;
    const unsigned char* src = D->base + (size_t)r * kRankBytes + FlagLayout::off_status * sizeof(uint64_t);
    const cudaError_t e = cudaMemcpy(&word, src, sizeof(word), cudaMemcpyDeviceToHost);  // pageable destination: nothing is allocated
    if (e != cudaSuccess) return fail(std::string("cudaMemcpy: ") + cudaGetErrorString(e));
    if (word != 0 && *code == 0) *code = (int)word;
  }
  return 0;
}

extern "C" int al_noalloc_reset(void* stream) {
  std::lock_guard<std::mutex> lock(g_mu);
  PerDevice* D = current_device_state();
  if (!D) return 1;
  const cudaError_t e = cudaMemsetAsync(D->base, 0, AL_NOALLOC_SCRATCH_BYTES, (cudaStream_t)stream);
  if (e != cudaSuccess) return fail(std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
  D->seq = 0;  // flags and epochs start over together
  return 0;
}
