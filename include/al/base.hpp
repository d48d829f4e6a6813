/**
 * @file base.hpp
 * Exceptions, the reduction-operator enum, the in-place sentinel and the
 * run-time datatype tags shared by every backend.
 *
 * Parity: include/aluminum/base.hpp:44-107 (al_exception, build_string,
 * throw_al_exception, terminate_al, ReductionOperator),
 * include/aluminum/internal.hpp:41-44 (IN_PLACE) and
 * include/aluminum/datatypes.hpp:35-56 (half / bfloat16 detection).
 *
 * Design difference: backends here are not header-only templates over T.  The
 * templated API in Al.hpp erases T into a DType tag and calls compiled
 * runtime functions, so that device kernels are instantiated once inside the
 * library instead of in every user translation unit.
 */
#pragma once

#include <cstddef>
#include <cstdint>
#include <cstring>
#include <exception>
#include <iostream>
#include <sstream>
#include <string>
#include <type_traits>

#include "al/config.hpp"

namespace Al {

/** Exception thrown by every failing library call. */
class al_exception : public std::exception {
 public:
  al_exception(const std::string& msg, const std::string& file, int line)
      : msg_(msg), file_(file), line_(line) {
    what_ = "Aluminum-B200 exception: " + file_ + ":" + std::to_string(line_) + " - " + msg_;
  }
  const char* what() const noexcept override { return what_.c_str(); }
  const std::string& message() const noexcept { return msg_; }

 private:
  std::string msg_, file_, what_;
  int line_;
};

/** Concatenate any streamable arguments into one string. */
template <typename... Args>
std::string build_string(Args&&... args) {
  std::ostringstream ss;
  (void)std::initializer_list<int>{((ss << std::forward<Args>(args)), 0)...};
  return ss.str();
}

#define throw_al_exception(...) \
  throw ::Al::al_exception(::Al::build_string(__VA_ARGS__), __FILE__, __LINE__)

/** For contexts that must not throw (destructors): report and terminate. */
#define terminate_al(...)                                                        \
  do {                                                                           \
    std::cerr << __FILE__ << ":" << __LINE__ << " - "                            \
              << ::Al::build_string(__VA_ARGS__) << std::endl;                   \
    std::terminate();                                                            \
  } while (0)

#define AL_IGNORE_NODISCARD(fn) \
  do { auto al_ignored_ = (fn); (void)al_ignored_; } while (0)

/** Element-wise reduction operators (same enumerators and order as the reference). */
enum class ReductionOperator : int {
  sum = 0, prod, min, max, lor, land, lxor, bor, band, bxor, avg
};

inline const char* reduction_name(ReductionOperator op) {
  switch (op) {
    case ReductionOperator::sum: return "sum";
    case ReductionOperator::prod: return "prod";
    case ReductionOperator::min: return "min";
    case ReductionOperator::max: return "max";
    case ReductionOperator::lor: return "lor";
    case ReductionOperator::land: return "land";
    case ReductionOperator::lxor: return "lxor";
    case ReductionOperator::bor: return "bor";
    case ReductionOperator::band: return "band";
    case ReductionOperator::bxor: return "bxor";
    case ReductionOperator::avg: return "avg";
  }
  return "unknown";
}

/** 16-bit storage types usable from plain host C++ (bit patterns only). */
struct half_t { uint16_t bits; };
struct bfloat16_t { uint16_t bits; };

/** Run-time datatype tag. The numeric values are part of the C API. */
enum class DType : int {
  i8 = 0, u8, i16, u16, i32, u32, i64, u64, f16, bf16, f32, f64, f128 /* long double, host only */,
  invalid = -1
};

constexpr size_t dtype_size(DType t) {
  switch (t) {
    case DType::i8: case DType::u8: return 1;
    case DType::i16: case DType::u16: case DType::f16: case DType::bf16: return 2;
    case DType::i32: case DType::u32: case DType::f32: return 4;
    case DType::i64: case DType::u64: case DType::f64: return 8;
    case DType::f128: return sizeof(long double);
    default: return 0;
  }
}

constexpr bool dtype_is_float(DType t) {
  return t == DType::f16 || t == DType::bf16 || t == DType::f32 || t == DType::f64 ||
         t == DType::f128;
}

inline const char* dtype_name(DType t) {
  switch (t) {
    case DType::i8: return "int8"; case DType::u8: return "uint8";
    case DType::i16: return "int16"; case DType::u16: return "uint16";
    case DType::i32: return "int32"; case DType::u32: return "uint32";
    case DType::i64: return "int64"; case DType::u64: return "uint64";
    case DType::f16: return "half"; case DType::bf16: return "bfloat16";
    case DType::f32: return "float"; case DType::f64: return "double";
    case DType::f128: return "long double";
    default: return "invalid";
  }
}

/** Compile-time map C++ type -> DType. Unsupported types map to DType::invalid. */
template <typename T, typename = void>
struct TypeMap { static constexpr DType value = DType::invalid; };

template <typename T>
struct TypeMap<T, std::enable_if_t<std::is_integral<T>::value && !std::is_same<T, bool>::value>> {
  static constexpr DType value =
      sizeof(T) == 1 ? (std::is_signed<T>::value ? DType::i8 : DType::u8)
    : sizeof(T) == 2 ? (std::is_signed<T>::value ? DType::i16 : DType::u16)
    : sizeof(T) == 4 ? (std::is_signed<T>::value ? DType::i32 : DType::u32)
                     : (std::is_signed<T>::value ? DType::i64 : DType::u64);
};
template <> struct TypeMap<float> { static constexpr DType value = DType::f32; };
template <> struct TypeMap<double> { static constexpr DType value = DType::f64; };
template <> struct TypeMap<long double> { static constexpr DType value = DType::f128; };
template <> struct TypeMap<half_t> { static constexpr DType value = DType::f16; };
template <> struct TypeMap<bfloat16_t> { static constexpr DType value = DType::bf16; };

/**
 * Specialise (or use AL_DECLARE_DTYPE) to teach the API about a foreign
 * 16-bit type such as __half or __nv_bfloat16; Al.hpp does so when the CUDA
 * headers are visible.
 */
#define AL_DECLARE_DTYPE(T, tag) \
  namespace Al { template <> struct TypeMap<T> { static constexpr DType value = tag; }; }

namespace internal {

/** Sentinel passed as the send buffer of an in-place operation. */
template <typename T>
inline T* IN_PLACE() { return reinterpret_cast<T*>(-1); }
inline const void* in_place_ptr() { return reinterpret_cast<const void*>(-1); }
inline bool is_in_place(const void* p) { return p == in_place_ptr(); }

}  // namespace internal
}  // namespace Al
