/**
 * @file traits.hpp
 * Compile-time capability tables: which operations, datatypes and reduction
 * operators each backend supports, plus classification of operations.
 * Parity: include/aluminum/traits/traits_base.hpp:43-214 and the per-backend
 * tables in mpi_traits.hpp:42-106, nccl_traits.hpp:41-103, ht_traits.hpp.
 */
#pragma once
#include <type_traits>

#include "al/base.hpp"

namespace Al {

class HostBackend;
class DeviceBackend;
class HostTransferBackend;

enum class AlOperation {
  allgather, allgatherv, allreduce, alltoall, alltoallv, barrier, bcast, gather, gatherv, reduce,
  reduce_scatter, reduce_scatterv, scatter, scatterv, send, recv, sendrecv, multisendrecv
};

constexpr const char* AlOperationName(AlOperation op) {
  switch (op) {
    case AlOperation::allgather: return "allgather"; case AlOperation::allgatherv: return "allgatherv";
    case AlOperation::allreduce: return "allreduce"; case AlOperation::alltoall: return "alltoall";
    case AlOperation::alltoallv: return "alltoallv"; case AlOperation::barrier: return "barrier";
    case AlOperation::bcast: return "bcast"; case AlOperation::gather: return "gather";
    case AlOperation::gatherv: return "gatherv"; case AlOperation::reduce: return "reduce";
    case AlOperation::reduce_scatter: return "reduce_scatter"; case AlOperation::reduce_scatterv: return "reduce_scatterv";
    case AlOperation::scatter: return "scatter"; case AlOperation::scatterv: return "scatterv";
    case AlOperation::send: return "send"; case AlOperation::recv: return "recv";
    case AlOperation::sendrecv: return "sendrecv"; case AlOperation::multisendrecv: return "multisendrecv";
  }
  return "unknown";
}

constexpr bool IsReductionOp(AlOperation op) {
  return op == AlOperation::allreduce || op == AlOperation::reduce || op == AlOperation::reduce_scatter ||
         op == AlOperation::reduce_scatterv;
}
constexpr bool IsVectorOp(AlOperation op) {
  return op == AlOperation::allgatherv || op == AlOperation::alltoallv || op == AlOperation::gatherv ||
         op == AlOperation::reduce_scatterv || op == AlOperation::scatterv;
}
constexpr bool IsPt2PtOp(AlOperation op) {
  return op == AlOperation::send || op == AlOperation::recv || op == AlOperation::sendrecv ||
         op == AlOperation::multisendrecv;
}
constexpr bool IsCollectiveOp(AlOperation op) { return !IsPt2PtOp(op); }
constexpr bool IsRootedOp(AlOperation op) {
  return op == AlOperation::bcast || op == AlOperation::gather || op == AlOperation::gatherv ||
         op == AlOperation::reduce || op == AlOperation::scatter || op == AlOperation::scatterv;
}

/** Every backend of this library implements every operation. */
template <AlOperation Op, typename Backend> struct IsOpSupported : std::true_type {};

/**
 * Operations with a real choice behind their `algo` argument: on the device backend allreduce
 * (one-shot / two-shot / NVLS) and the four operations that can run on registered buffers
 * (staged / window).  The enum itself is OpAlgoType<Op, Backend>::type, defined with the backends.
 */
template <AlOperation Op, typename Backend> struct OpSupportsAlgos : std::false_type {};
template <> struct OpSupportsAlgos<AlOperation::allreduce, DeviceBackend> : std::true_type {};
template <> struct OpSupportsAlgos<AlOperation::reduce_scatter, DeviceBackend> : std::true_type {};
template <> struct OpSupportsAlgos<AlOperation::allgather, DeviceBackend> : std::true_type {};
template <> struct OpSupportsAlgos<AlOperation::alltoall, DeviceBackend> : std::true_type {};
template <> struct OpSupportsAlgos<AlOperation::bcast, DeviceBackend> : std::true_type {};
template <AlOperation Op, typename Backend> struct OpAlgoType;

template <typename Backend> struct AlBackendName;
template <> struct AlBackendName<HostBackend> { static constexpr const char* value = "host"; };
template <> struct AlBackendName<DeviceBackend> { static constexpr const char* value = "device"; };
template <> struct AlBackendName<HostTransferBackend> { static constexpr const char* value = "ht"; };

namespace internal {
constexpr bool device_dtype(DType t) { return t != DType::invalid && t != DType::f128; }
}

/** Host and host-transfer: every mapped type incl. long double; device: all but long double. */
template <typename Backend, typename T> struct IsTypeSupported
    : std::integral_constant<bool, TypeMap<T>::value != DType::invalid> {};
template <typename T> struct IsTypeSupported<DeviceBackend, T>
    : std::integral_constant<bool, internal::device_dtype(TypeMap<T>::value)> {};

/** Run-time form: bitwise operators need an integer type; everything else is supported everywhere. */
constexpr bool reduction_supported(DType dt, ReductionOperator op) {
  return !((op == ReductionOperator::bor || op == ReductionOperator::band || op == ReductionOperator::bxor) &&
           dtype_is_float(dt));
}
/** Is the operator available on the backend for at least one datatype?  (All are, everywhere.) */
template <typename Backend, ReductionOperator Op> struct IsReductionOpSupported : std::true_type {};
/**
 * The table that matches what the kernels and host loops accept: operator x datatype x backend.
 * Bitwise operators need an integer type on every backend; everything else is available wherever the
 * datatype is.  Al::Allreduce & co. throw the same verdict at run time (the operator is a run-time
 * argument), so `IsReductionSupported<B, float, bor>` being false is what a caller can test up front.
 */
template <typename Backend, typename T, ReductionOperator Op> struct IsReductionSupported
    : std::integral_constant<bool, IsTypeSupported<Backend, T>::value && reduction_supported(TypeMap<T>::value, Op)> {};

static_assert(IsReductionOp(AlOperation::reduce_scatterv) && IsVectorOp(AlOperation::reduce_scatterv), "traits");
static_assert(IsRootedOp(AlOperation::bcast) && !IsRootedOp(AlOperation::allreduce), "traits");
static_assert(IsTypeSupported<HostBackend, long double>::value, "traits");
static_assert(!IsTypeSupported<DeviceBackend, long double>::value, "traits");
static_assert(IsTypeSupported<DeviceBackend, float>::value && IsTypeSupported<DeviceBackend, bfloat16_t>::value, "traits");
static_assert(!IsReductionSupported<DeviceBackend, float, ReductionOperator::bor>::value, "traits");
static_assert(IsReductionSupported<DeviceBackend, int, ReductionOperator::bor>::value, "traits");
static_assert(IsReductionSupported<DeviceBackend, float, ReductionOperator::avg>::value, "traits");
static_assert(!IsReductionSupported<DeviceBackend, long double, ReductionOperator::sum>::value, "traits");
static_assert(IsReductionSupported<HostBackend, long double, ReductionOperator::sum>::value, "traits");
static_assert(OpSupportsAlgos<AlOperation::allgather, DeviceBackend>::value && !OpSupportsAlgos<AlOperation::gather, DeviceBackend>::value, "traits");

}  // namespace Al
