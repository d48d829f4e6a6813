/**
 * @file reduce.hpp
 * Type-erased element-wise reductions on host memory, including IEEE half and
 * bfloat16 (stored as 16-bit patterns, accumulated in fp32).
 *
 * Parity: the reference reduces on the host through MPI_Op, with custom
 * MPI_Ops for the two 16-bit float types that accumulate pairwise in fp32
 * (src/mpi_impl.cpp:61-145, include/aluminum/mpi/utils.hpp:195-256).  Here
 * all contributions of one element are folded in rank order in a wide
 * accumulator and rounded once, so every rank obtains bit-identical results.
 */
#pragma once
#include <cstddef>

#include "al/base.hpp"

namespace Al {
namespace internal {
namespace host {

float half_to_float(uint16_t h);
uint16_t float_to_half(float f);
inline float bf16_to_float(uint16_t b) {
  uint32_t u = (uint32_t)b << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
uint16_t float_to_bf16(float f);

/** True when `op` is defined for `dt` (bitwise operators need an integer type). */
bool reduction_supported(DType dt, ReductionOperator op);

/**
 * out[i] = op(srcs[0][i], srcs[1][i], ..., srcs[nsrc-1][i]) for i in [0, n).
 * `out` may alias any source.  For ReductionOperator::avg the sum is divided
 * by `nsrc`.
 */
void reduce_multi(DType dt, ReductionOperator op, void* out, const void* const* srcs, int nsrc, size_t n);

}  // namespace host
}  // namespace internal
}  // namespace Al
