// CTA-wide copy, convert and multi-source reduce loops used by the collective
// kernels.  Reads of staging memory (local or a peer's) bypass L1 (ld.cg), so a
// line cached during an earlier operation can never be served stale.
#pragma once
#include "common.cuh"

namespace Al {
namespace internal {
namespace device {

// ---------------------------------------------------------------------------
// element traits: accumulator type and conversions
// ---------------------------------------------------------------------------
template <typename T> struct Elem { using Acc = T; static __device__ __forceinline__ Acc up(T v) { return v; } static __device__ __forceinline__ T down(Acc a) { return a; } };
template <> struct Elem<__half> {
  using Acc = float;
  static __device__ __forceinline__ float up(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half down(float a) { return __float2half_rn(a); }
};
template <> struct Elem<__nv_bfloat16> {
  using Acc = float;
  static __device__ __forceinline__ float up(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 down(float a) { return __float2bfloat16_rn(a); }
};

/** Convert between accumulator types (float <-> float only in practice). */
template <typename To, typename From>
__device__ __forceinline__ To acc_cast(From v) { return (To)v; }

// ---------------------------------------------------------------------------
// reduction functors on accumulator values
// ---------------------------------------------------------------------------
struct RedSum { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return a + b; } };
struct RedMin { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return b < a ? b : a; } };
struct RedMax { template <typename A> __device__ __forceinline__ A operator()(A a, A b) const { return a < b ? b : a; } };
struct RedNone { template <typename A> __device__ __forceinline__ A operator()(A a, A) const { return a; } };

template <typename A, bool IsInt = std::is_integral<A>::value>
struct BitOps {
  static __device__ __forceinline__ A apply(int, A a, A) { return a; }
};
template <typename A>
struct BitOps<A, true> {
  static __device__ __forceinline__ A apply(int op, A a, A b) {
    switch ((ReductionOperator)op) {
      case ReductionOperator::bor: return (A)(a | b);
      case ReductionOperator::band: return (A)(a & b);
      case ReductionOperator::bxor: return (A)(a ^ b);
      default: return a;
    }
  }
};

/** Operator chosen at run time (integer types and the less common operators). */
struct RedRuntime {
  int op;
  template <typename A>
  __device__ __forceinline__ A operator()(A a, A b) const {
    switch ((ReductionOperator)op) {
      case ReductionOperator::sum:
      case ReductionOperator::avg: return a + b;
      case ReductionOperator::prod: return a * b;
      case ReductionOperator::min: return b < a ? b : a;
      case ReductionOperator::max: return a < b ? b : a;
      case ReductionOperator::lor: return (A)((a != A(0)) || (b != A(0)));
      case ReductionOperator::land: return (A)((a != A(0)) && (b != A(0)));
      case ReductionOperator::lxor: return (A)((a != A(0)) != (b != A(0)));
      default: return BitOps<A>::apply(op, a, b);
    }
  }
};

// ---------------------------------------------------------------------------
// work split
// ---------------------------------------------------------------------------
/** Sub-range [lo, hi) of [0, len) owned by part `i` of `n`, boundaries multiples of `align`. */
__device__ __forceinline__ void split_range(size_t len, unsigned i, unsigned n, size_t align, size_t& lo, size_t& hi) {
  size_t per = (len + n - 1) / n;
  per = (per + align - 1) / align * align;
  lo = per * i;
  if (lo > len) lo = len;
  hi = lo + per;
  if (hi > len) hi = len;
}

__device__ __forceinline__ size_t clamp_len(size_t count, size_t lo, size_t cap) {
  if (count <= lo) return 0;
  const size_t r = count - lo;
  return r < cap ? r : cap;
}

// ---------------------------------------------------------------------------
// copies
// ---------------------------------------------------------------------------
template <typename V>
__device__ __forceinline__ void copy_units(char* dst, const char* src, size_t units, bool src_is_staging,
                                           unsigned lane, unsigned nlanes) {
  V* d = (V*)dst;
  const V* s = (const V*)src;
  const size_t stride = nlanes;
  size_t i = lane;
  // four independent loads in flight per thread
  for (; i + 3 * stride < units; i += 4 * stride) {
    V a, b, c, e;
    if (src_is_staging) { a = __ldcg(s + i); b = __ldcg(s + i + stride); c = __ldcg(s + i + 2 * stride); e = __ldcg(s + i + 3 * stride); }
    else { a = s[i]; b = s[i + stride]; c = s[i + 2 * stride]; e = s[i + 3 * stride]; }
    d[i] = a; d[i + stride] = b; d[i + 2 * stride] = c; d[i + 3 * stride] = e;
  }
  for (; i < units; i += stride) d[i] = src_is_staging ? __ldcg(s + i) : s[i];
}

/**
 * Copy `nbytes` with `nlanes` cooperating threads (this thread is `lane`).  Uses
 * the widest unit both addresses allow (16, 8, 4, 2 or 1 bytes).
 */
__device__ __forceinline__ void group_copy(char* dst, const char* src, size_t nbytes, bool src_is_staging,
                                           unsigned lane, unsigned nlanes) {
  if (nbytes == 0) return;
  const uintptr_t mis = (uintptr_t)dst | (uintptr_t)src;
  if ((mis & 15) == 0) {
    const size_t nv = nbytes >> 4;
    copy_units<uint4>(dst, src, nv, src_is_staging, lane, nlanes);
    const size_t done = nv << 4;
    for (size_t k = lane; k < nbytes - done; k += nlanes) dst[done + k] = src[done + k];
  } else if ((mis & 7) == 0) {
    const size_t nv = nbytes >> 3;
    copy_units<uint2>(dst, src, nv, src_is_staging, lane, nlanes);
    const size_t done = nv << 3;
    for (size_t k = lane; k < nbytes - done; k += nlanes) dst[done + k] = src[done + k];
  } else if ((mis & 3) == 0) {
    const size_t nv = nbytes >> 2;
    copy_units<uint32_t>(dst, src, nv, src_is_staging, lane, nlanes);
    const size_t done = nv << 2;
    for (size_t k = lane; k < nbytes - done; k += nlanes) dst[done + k] = src[done + k];
  } else if ((mis & 1) == 0) {
    const size_t nv = nbytes >> 1;
    copy_units<uint16_t>(dst, src, nv, src_is_staging, lane, nlanes);
    if ((nbytes & 1) && lane == 0) dst[nbytes - 1] = src[nbytes - 1];
  } else {
    copy_units<uint8_t>(dst, src, nbytes, src_is_staging, lane, nlanes);
  }
}

/** Copy with all threads of the CTA. */
__device__ __forceinline__ void cta_copy(char* dst, const char* src, size_t nbytes, bool src_is_staging) {
  group_copy(dst, src, nbytes, src_is_staging, threadIdx.x, blockDim.x);
}

// ---------------------------------------------------------------------------
// publish: one local source, several (possibly remote) destinations
// ---------------------------------------------------------------------------
template <typename V>
__device__ __forceinline__ void fanout_units(char* const* dsts, int ndst, size_t dst_off, const char* src, size_t units) {
  const V* s = (const V*)src;
  const size_t stride = blockDim.x;
  size_t i = threadIdx.x;
  for (; i + 3 * stride < units; i += 4 * stride) {
    const V a = s[i], b = s[i + stride], c = s[i + 2 * stride], e = s[i + 3 * stride];
#pragma unroll
    for (int d = 0; d < kMaxRanks; ++d) {
      if (d < ndst) {
        V* o = (V*)(dsts[d] + dst_off);
        o[i] = a; o[i + stride] = b; o[i + 2 * stride] = c; o[i + 3 * stride] = e;
      }
    }
  }
  for (; i < units; i += stride) {
    const V a = s[i];
#pragma unroll
    for (int d = 0; d < kMaxRanks; ++d)
      if (d < ndst) ((V*)(dsts[d] + dst_off))[i] = a;
  }
}

/**
 * Store `nbytes` read once from local `src` at byte offset `dst_off` of each of
 * `ndst` staging bases (peer-mapped memory: plain stores over NVLink, which do
 * not stall the issuing thread the way remote loads do).
 */
__device__ __forceinline__ void cta_fanout(char* const* dsts, int ndst, size_t dst_off, const char* src, size_t nbytes) {
  if (nbytes == 0 || ndst == 0) return;
  const uintptr_t mis = (uintptr_t)src | (uintptr_t)dst_off;  // staging bases are 256-byte aligned
  if ((mis & 15) == 0) {
    const size_t nv = nbytes >> 4;
    fanout_units<uint4>(dsts, ndst, dst_off, src, nv);
    const size_t done = nv << 4;
    if (threadIdx.x < (nbytes - done))
      for (int d = 0; d < ndst; ++d) dsts[d][dst_off + done + threadIdx.x] = src[done + threadIdx.x];
  } else if ((mis & 3) == 0) {
    const size_t nv = nbytes >> 2;
    fanout_units<uint32_t>(dsts, ndst, dst_off, src, nv);
    const size_t done = nv << 2;
    if (threadIdx.x < (nbytes - done))
      for (int d = 0; d < ndst; ++d) dsts[d][dst_off + done + threadIdx.x] = src[done + threadIdx.x];
  } else if ((mis & 1) == 0) {
    const size_t nv = nbytes >> 1;
    fanout_units<uint16_t>(dsts, ndst, dst_off, src, nv);
    if ((nbytes & 1) && threadIdx.x == 0)
      for (int d = 0; d < ndst; ++d) dsts[d][dst_off + nbytes - 1] = src[nbytes - 1];
  } else {
    fanout_units<uint8_t>(dsts, ndst, dst_off, src, nbytes);
  }
}

/** Single destination, a subset of the CTA's threads: used to serve all peers of a small message at once. */
template <typename Ti, typename Tw>
__device__ __forceinline__ void group_publish(char* dst, const Ti* src, size_t n, unsigned lane, unsigned nlanes) {
  if constexpr (std::is_same<Ti, Tw>::value) {
    group_copy(dst, (const char*)src, n * sizeof(Ti), false, lane, nlanes);
  } else {
    using Ai = typename Elem<Ti>::Acc;
    using Aw = typename Elem<Tw>::Acc;
    for (size_t i = lane; i < n; i += nlanes) ((Tw*)dst)[i] = Elem<Tw>::down(acc_cast<Aw, Ai>(Elem<Ti>::up(src[i])));
  }
}

/** Publish n elements of user type Ti as wire type Tw into every destination (cast fused in). */
template <typename Ti, typename Tw>
__device__ __forceinline__ void cta_publish(char* const* dsts, int ndst, size_t dst_off, const Ti* src, size_t n) {
  if constexpr (std::is_same<Ti, Tw>::value) {
    cta_fanout(dsts, ndst, dst_off, (const char*)src, n * sizeof(Ti));
  } else {
    using Ai = typename Elem<Ti>::Acc;
    using Aw = typename Elem<Tw>::Acc;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
      const Tw v = Elem<Tw>::down(acc_cast<Aw, Ai>(Elem<Ti>::up(src[i])));
#pragma unroll
      for (int d = 0; d < kMaxRanks; ++d)
        if (d < ndst) ((Tw*)(dsts[d] + dst_off))[i] = v;
    }
  }
}

/** dst[i] = (Tw)src[i] for i in [0, n): the publish step of an operation whose wire type differs. */
template <typename Ti, typename Tw>
__device__ __forceinline__ void cta_convert(Tw* dst, const Ti* src, size_t n) {
  if constexpr (std::is_same<Ti, Tw>::value) {
    cta_copy((char*)dst, (const char*)src, n * sizeof(Ti), false);
  } else {
    using Ai = typename Elem<Ti>::Acc;
    using Aw = typename Elem<Tw>::Acc;
    for (size_t i = threadIdx.x; i < n; i += blockDim.x)
      dst[i] = Elem<Tw>::down(acc_cast<Aw, Ai>(Elem<Ti>::up(src[i])));
  }
}

// ---------------------------------------------------------------------------
// multi-source reduction
// ---------------------------------------------------------------------------
template <typename A>
__device__ __forceinline__ A finish_acc(A a, double scale, int int_div) {
  if constexpr (std::is_integral<A>::value) {
    return int_div > 1 ? (A)(a / (A)int_div) : a;
  } else {
    return scale != 1.0 ? (A)(a * (A)scale) : a;
  }
}

/**
 * out[i] = finish(red(src_0[i], src_1[i], ..., src_{p-1}[i])) for i in [0, n),
 * where src_r = (const Tw*)(bases[r] + byte_off), written to each of the `ndst`
 * destinations dsts[d] (all holding To elements; several destinations are used
 * when a reduced slice is pushed to every peer).  Sources are staging memory
 * (16-byte aligned); contributions are folded in rank order so every rank
 * computes bit-identical results.  A destination may alias one of the sources.  Sources that are
 * not 16-byte aligned are read element by element.
 */
template <typename Tw, typename To, typename Red>
__device__ __forceinline__ void cta_reduce(To* const* dsts, int ndst, char* const* bases, size_t byte_off, int p,
                                           size_t n, Red red, double scale, int int_div) {
  using Aw = typename Elem<Tw>::Acc;
  using Ao = typename Elem<To>::Acc;
  constexpr int VEC = 16 / (int)sizeof(Tw);
  constexpr size_t out_bytes = (size_t)VEC * sizeof(To);
  constexpr size_t out_align = out_bytes < 16 ? out_bytes : 16;
  bool aligned = true;
  for (int d = 0; d < ndst; ++d) aligned = aligned && ((uintptr_t)dsts[d] % out_align == 0);
  // staging sources always are 16-byte aligned; registered user buffers (window kernels) need not be
  for (int r = 0; r < p; ++r) aligned = aligned && ((uintptr_t)(bases[r] + byte_off) % 16 == 0);
  const size_t nvec = aligned ? n / VEC : 0;
  union InPack { uint4 u; Tw e[VEC]; };
  union OutPack { uint4 u[(out_bytes + 15) / 16]; To e[VEC]; };

  auto store = [&](size_t v, const OutPack& o) {
#pragma unroll
    for (int d = 0; d < kMaxRanks; ++d) {
      if (d < ndst) {
        To* dst = dsts[d];
        if constexpr (out_bytes >= 16) {
#pragma unroll
          for (int q = 0; q < (int)(out_bytes / 16); ++q) ((uint4*)dst)[v * (out_bytes / 16) + q] = o.u[q];
        } else if constexpr (out_bytes == 8) {
          ((uint2*)dst)[v] = *(const uint2*)&o.u[0];
        } else {
          ((uint32_t*)dst)[v] = *(const uint32_t*)&o.u[0];
        }
      }
    }
  };

  for (size_t v = threadIdx.x; v < nvec; v += 2 * (size_t)blockDim.x) {
    const size_t v2 = v + blockDim.x;
    const bool has2 = v2 < nvec;
    Aw acc0[VEC], acc1[VEC];
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < p) {
        const uint4* s = (const uint4*)(bases[r] + byte_off);
        InPack a, b;
        a.u = __ldcg(s + v);
        if (has2) b.u = __ldcg(s + v2);
#pragma unroll
        for (int k = 0; k < VEC; ++k) {
          const Aw x = Elem<Tw>::up(a.e[k]);
          acc0[k] = r == 0 ? x : red(acc0[k], x);
          if (has2) {
            const Aw y = Elem<Tw>::up(b.e[k]);
            acc1[k] = r == 0 ? y : red(acc1[k], y);
          }
        }
      }
    }
    OutPack o;
#pragma unroll
    for (int k = 0; k < VEC; ++k) o.e[k] = Elem<To>::down(acc_cast<Ao, Aw>(finish_acc(acc0[k], scale, int_div)));
    store(v, o);
    if (has2) {
#pragma unroll
      for (int k = 0; k < VEC; ++k) o.e[k] = Elem<To>::down(acc_cast<Ao, Aw>(finish_acc(acc1[k], scale, int_div)));
      store(v2, o);
    }
  }
  // scalar remainder (and the whole range when a destination is not aligned for vector stores)
  for (size_t i = nvec * VEC + threadIdx.x; i < n; i += blockDim.x) {
    Aw acc = Aw();
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) {
      if (r < p) {
        const Aw x = Elem<Tw>::up(__ldcg((const Tw*)(bases[r] + byte_off) + i));
        acc = r == 0 ? x : red(acc, x);
      }
    }
    const To out = Elem<To>::down(acc_cast<Ao, Aw>(finish_acc(acc, scale, int_div)));
    for (int d = 0; d < ndst; ++d) dsts[d][i] = out;
  }
}

}  // namespace device
}  // namespace internal
}  // namespace Al
