// Host-side element-wise reductions (see al/host/reduce.hpp).
#include "al/host/reduce.hpp"

#include <algorithm>
#include <cmath>

namespace Al {
namespace internal {
namespace host {

float half_to_float(uint16_t h) {
  const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {  // subnormal: renormalise
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      u = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

uint16_t float_to_half(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint32_t sign = (u >> 16) & 0x8000u;
  const uint32_t absu = u & 0x7fffffffu;
  if (absu >= 0x7f800000u) {  // inf / nan
    return (uint16_t)(sign | 0x7c00u | ((absu > 0x7f800000u) ? 0x200u : 0));
  }
  if (absu >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to inf
  if (absu < 0x33000001u) return (uint16_t)sign;                // rounds to zero
  int32_t exp = (int32_t)(absu >> 23) - 127 + 15;
  uint32_t man = absu & 0x7fffffu;
  if (exp <= 0) {  // subnormal half
    man |= 0x800000u;
    const int shift = 14 - exp;  // 13 + (1 - exp)
    uint32_t hm = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1);
    const uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (hm & 1))) ++hm;
    return (uint16_t)(sign | hm);
  }
  uint32_t hm = man >> 13;
  const uint32_t rem = man & 0x1fffu;
  uint32_t h = ((uint32_t)exp << 10) | hm;
  if (rem > 0x1000u || (rem == 0x1000u && (hm & 1))) ++h;  // carries into the exponent correctly
  return (uint16_t)(sign | h);
}

uint16_t float_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);  // quiet NaN
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;  // round to nearest even
  return (uint16_t)(u >> 16);
}

bool reduction_supported(DType dt, ReductionOperator op) {
  if (dt == DType::invalid) return false;
  const bool bitwise = op == ReductionOperator::bor || op == ReductionOperator::band ||
                       op == ReductionOperator::bxor;
  if (bitwise && dtype_is_float(dt)) return false;
  return true;
}

namespace {

template <typename A>
inline A apply(ReductionOperator op, A a, A b) {
  switch (op) {
    case ReductionOperator::sum:
    case ReductionOperator::avg: return a + b;
    case ReductionOperator::prod: return a * b;
    case ReductionOperator::min: return b < a ? b : a;
    case ReductionOperator::max: return a < b ? b : a;
    case ReductionOperator::lor: return (A)((a != A(0)) || (b != A(0)));
    case ReductionOperator::land: return (A)((a != A(0)) && (b != A(0)));
    case ReductionOperator::lxor: return (A)((a != A(0)) != (b != A(0)));
    default: return a;
  }
}

template <typename A>
inline A apply_bits(ReductionOperator op, A a, A b) {
  switch (op) {
    case ReductionOperator::bor: return (A)(a | b);
    case ReductionOperator::band: return (A)(a & b);
    case ReductionOperator::bxor: return (A)(a ^ b);
    default: return apply<A>(op, a, b);
  }
}

// T = storage type, A = accumulator, with loaders/storers for the 16-bit floats.
template <typename T, typename A, typename Load, typename Store, bool Bits>
void reduce_impl(ReductionOperator op, void* out, const void* const* srcs, int nsrc, size_t n,
                 Load load, Store store) {
  T* o = (T*)out;
  const bool logical = op == ReductionOperator::lor || op == ReductionOperator::land ||
                       op == ReductionOperator::lxor;
  for (size_t i = 0; i < n; ++i) {
    A acc = load(((const T*)srcs[0])[i]);
    if (logical && nsrc == 1) acc = (A)(acc != A(0));
    for (int r = 1; r < nsrc; ++r) {
      A v = load(((const T*)srcs[r])[i]);
      if constexpr (Bits) acc = apply_bits<A>(op, acc, v);
      else acc = apply<A>(op, acc, v);
    }
    if (op == ReductionOperator::avg) acc = (A)(acc / (A)nsrc);
    o[i] = store(acc);
  }
}

template <typename T>
void reduce_int(ReductionOperator op, void* out, const void* const* srcs, int nsrc, size_t n) {
  reduce_impl<T, T, T (*)(T), T (*)(T), true>(
      op, out, srcs, nsrc, n, +[](T v) { return v; }, +[](T v) { return v; });
}
template <typename T>
void reduce_flt(ReductionOperator op, void* out, const void* const* srcs, int nsrc, size_t n) {
  reduce_impl<T, T, T (*)(T), T (*)(T), false>(
      op, out, srcs, nsrc, n, +[](T v) { return v; }, +[](T v) { return v; });
}

}  // namespace

void reduce_multi(DType dt, ReductionOperator op, void* out, const void* const* srcs, int nsrc, size_t n) {
  if (!reduction_supported(dt, op))
    throw_al_exception("reduction ", reduction_name(op), " is not defined for ", dtype_name(dt));
  if (nsrc < 1) throw_al_exception("reduce_multi needs at least one source");
  switch (dt) {
    case DType::i8: reduce_int<int8_t>(op, out, srcs, nsrc, n); break;
    case DType::u8: reduce_int<uint8_t>(op, out, srcs, nsrc, n); break;
    case DType::i16: reduce_int<int16_t>(op, out, srcs, nsrc, n); break;
    case DType::u16: reduce_int<uint16_t>(op, out, srcs, nsrc, n); break;
    case DType::i32: reduce_int<int32_t>(op, out, srcs, nsrc, n); break;
    case DType::u32: reduce_int<uint32_t>(op, out, srcs, nsrc, n); break;
    case DType::i64: reduce_int<int64_t>(op, out, srcs, nsrc, n); break;
    case DType::u64: reduce_int<uint64_t>(op, out, srcs, nsrc, n); break;
    case DType::f32: reduce_flt<float>(op, out, srcs, nsrc, n); break;
    case DType::f64: reduce_flt<double>(op, out, srcs, nsrc, n); break;
    case DType::f128: reduce_flt<long double>(op, out, srcs, nsrc, n); break;
    case DType::f16:
      reduce_impl<uint16_t, float, float (*)(uint16_t), uint16_t (*)(float), false>(
          op, out, srcs, nsrc, n, &half_to_float, &float_to_half);
      break;
    case DType::bf16:
      reduce_impl<uint16_t, float, float (*)(uint16_t), uint16_t (*)(float), false>(
          op, out, srcs, nsrc, n, +[](uint16_t b) { return bf16_to_float(b); }, &float_to_bf16);
      break;
    default: throw_al_exception("unsupported datatype");
  }
}

}  // namespace host
}  // namespace internal
}  // namespace Al
