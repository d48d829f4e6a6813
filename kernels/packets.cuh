// Low-latency packets: 16-byte vectors {word, epoch, word, epoch} that carry their own arrival signal.
// A vector's two 8-byte halves are each delivered whole, so a receiver that sees the expected epoch next to
// a word knows that the word is the sender's.  Used by the small collectives (ll.cu) and by small
// point-to-point messages (p2p.cu).  Every poll is bounded.
#pragma once
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

__device__ __forceinline__ void st_packet(char* dst, uint32_t a, uint32_t b, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(a), "r"(flag), "r"(b), "r"(flag) : "memory");
}
__device__ __forceinline__ uint4 ld_packet(const char* src) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src) : "memory");
  return v;
}

/** 16 bytes of payload starting at element `e0` of `src` (zeros beyond `n`), whatever the alignment. */
template <typename T>
__device__ __forceinline__ uint4 load_group(const T* src, size_t e0, size_t n) {
  constexpr int VEC = 16 / (int)sizeof(T);
  union { uint4 u; T e[VEC]; } x;
  const T* p = src + e0;
  if (e0 + VEC <= n && ((uintptr_t)p & 15) == 0) {
    x.u = *(const uint4*)p;
  } else {
    x.u = uint4{0, 0, 0, 0};
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      if (e0 + k < n) x.e[k] = p[k];
  }
  return x.u;
}

template <typename T>
__device__ __forceinline__ void store_group(T* dst, size_t e0, size_t n, uint4 v) {
  constexpr int VEC = 16 / (int)sizeof(T);
  union { uint4 u; T e[VEC]; } x;
  x.u = v;
  T* p = dst + e0;
  if (e0 + VEC <= n && ((uintptr_t)p & 15) == 0) {
    *(uint4*)p = v;
  } else {
#pragma unroll
    for (int k = 0; k < VEC; ++k)
      if (e0 + k < n) p[k] = x.e[k];
  }
}

__device__ __forceinline__ void send_group(char* slot, size_t g, uint4 v, uint32_t flag) {
  st_packet(slot + g * 32, v.x, v.y, flag);
  st_packet(slot + g * 32 + 16, v.z, v.w, flag);
}

/** Poll group g of a slot until all four packets carry `flag`.  false = timed out (reported). */
__device__ __forceinline__ bool recv_group(const char* slot, size_t g, uint32_t flag, uint4& out, const Workspace& ws,
                                           int rank, int peer, uint64_t epoch, uint64_t timeout_ns, uint32_t where = 4) {
  unsigned spins = 0;
  uint64_t t0 = 0;
  for (;;) {
    const uint4 a = ld_packet(slot + g * 32), b = ld_packet(slot + g * 32 + 16);
    if (a.y == flag && a.w == flag && b.y == flag && b.w == flag) {
      out = uint4{a.x, a.z, b.x, b.z};
      return true;
    }
    if (++spins > 64) {
      __nanosleep(spins > 8192 ? 200 : 20);
      if (t0 == 0) t0 = global_ns();
      else if ((spins & 127) == 0 && global_ns() - t0 > timeout_ns) {
        report_timeout(ws, rank, peer, where, epoch, a.y);
        return false;
      }
    }
  }
}

}  // namespace device
}  // namespace internal
}  // namespace Al
