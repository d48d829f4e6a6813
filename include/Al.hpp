/**
 * @file Al.hpp
 * Public C++ API: free function templates `Al::Op<Backend>(..., comm)`.
 *
 * Surface and semantics follow the reference's include/Al.hpp:73-2001: every
 * collective and point-to-point operation in blocking and Nonblocking* form,
 * out-of-place and in-place, with counts in elements, vector variants taking
 * std::vector<size_t> counts / displacements by value, `algo` as the last
 * defaulted argument, and Test / Wait on a backend-specific request.  Each
 * entry point runs the debug argument checks, opens a profiler scope, records
 * the call in the trace and hands a resolved description to the backend.
 *
 * Backends: Al::HostBackend (CPU ranks over shared memory), Al::DeviceBackend
 * (sm_100a kernels over NVLink), Al::HostTransferBackend (GPU buffers staged
 * through pinned host memory), and the Al::ext RMA interface on device
 * communicators.
 */
#pragma once
#include <vector>

#include "al/base.hpp"
#include "al/debug.hpp"
#include "al/host_backend.hpp"
#include "al/profiling.hpp"
#include "al/resolve.hpp"
#include "al/runtime.hpp"
#include "al/trace.hpp"
#include "al/traits.hpp"
#ifdef AL_HAS_CUDA
#include "al/device_backend.hpp"
#include "al/ht_backend.hpp"
#include "al/rma.hpp"
#endif

namespace Al {

// Algorithm enum of an operation on a backend (include/aluminum/traits/traits_base.hpp:186-214 of the reference).
template <AlOperation Op> struct OpAlgoType<Op, HostBackend> { using type = HostAlgo; };
#ifdef AL_HAS_CUDA
template <AlOperation Op> struct OpAlgoType<Op, HostTransferBackend> { using type = HostAlgo; };
template <AlOperation Op> struct OpAlgoType<Op, DeviceBackend> { using type = DeviceAlgo; };
template <> struct OpAlgoType<AlOperation::allreduce, DeviceBackend> { using type = DeviceAllreduceAlgo; };
static_assert(std::is_same<OpAlgoType<AlOperation::allgather, DeviceBackend>::type, DeviceBackend::allgather_algo_type>::value, "traits");
static_assert(std::is_same<OpAlgoType<AlOperation::allreduce, DeviceBackend>::type, DeviceBackend::allreduce_algo_type>::value, "traits");
#endif


namespace internal {
template <typename T>
constexpr DType dtype_of() {
  static_assert(TypeMap<T>::value != DType::invalid, "datatype not supported by Aluminum-B200");
  return TypeMap<T>::value;
}
template <typename Backend, typename T>
inline void api_enter(const char* name, const typename Backend::comm_type& comm) {
  if (trace::enabled()) trace::record_op(Backend::Name().c_str(), dtype_of<T>(), name, comm.rank(), comm.size());
}
}  // namespace internal

#define AL_API_ENTER(name)          \
  AL_API_SCOPE(name);               \
  internal::api_enter<Backend, T>(name, comm)

// ============================ Allreduce =====================================
template <typename Backend, typename T>
void Allreduce(const T* sendbuf, T* recvbuf, size_t count, ReductionOperator op, typename Backend::comm_type& comm,
               typename Backend::allreduce_algo_type algo = Backend::allreduce_algo_type::automatic) {
  AL_API_ENTER("allreduce");
  if (!reduction_supported(internal::dtype_of<T>(), op))
    throw_al_exception("allreduce: operator ", reduction_name(op), " is not defined for ", dtype_name(internal::dtype_of<T>()));
  debug::check_buffer(sendbuf, count); debug::check_buffer(recvbuf, count);
  internal::Resolved r = internal::resolve_uniform(internal::OpKind::allreduce, internal::dtype_of<T>(), sendbuf, recvbuf, count, op, 0, comm.rank(), comm.size());
  debug::check_resolved(r, r.send != nullptr, r.recv != nullptr, comm.rank(), comm.size());
  Backend::run_allreduce(std::move(r), comm, nullptr, algo);
}
template <typename Backend, typename T>
void Allreduce(T* buffer, size_t count, ReductionOperator op, typename Backend::comm_type& comm,
               typename Backend::allreduce_algo_type algo = Backend::allreduce_algo_type::automatic) {
  Allreduce<Backend, T>(internal::IN_PLACE<T>(), buffer, count, op, comm, algo);
}
template <typename Backend, typename T>
void NonblockingAllreduce(const T* sendbuf, T* recvbuf, size_t count, ReductionOperator op, typename Backend::comm_type& comm,
                          typename Backend::req_type& req,
                          typename Backend::allreduce_algo_type algo = Backend::allreduce_algo_type::automatic) {
  AL_API_ENTER("nonblocking-allreduce");
  if (!reduction_supported(internal::dtype_of<T>(), op))
    throw_al_exception("allreduce: operator ", reduction_name(op), " is not defined for ", dtype_name(internal::dtype_of<T>()));
  debug::check_buffer(sendbuf, count); debug::check_buffer(recvbuf, count);
  internal::Resolved r = internal::resolve_uniform(internal::OpKind::allreduce, internal::dtype_of<T>(), sendbuf, recvbuf, count, op, 0, comm.rank(), comm.size());
  debug::check_resolved(r, r.send != nullptr, r.recv != nullptr, comm.rank(), comm.size());
  Backend::run_allreduce(std::move(r), comm, &req, algo);
}
template <typename Backend, typename T>
void NonblockingAllreduce(T* buffer, size_t count, ReductionOperator op, typename Backend::comm_type& comm,
                          typename Backend::req_type& req,
                          typename Backend::allreduce_algo_type algo = Backend::allreduce_algo_type::automatic) {
  NonblockingAllreduce<Backend, T>(internal::IN_PLACE<T>(), buffer, count, op, comm, req, algo);
}

// ============================ generic helpers ================================
namespace internal {
/** Shared body of every uniform collective except allreduce (which carries an algorithm). */
template <typename Backend, typename T>
void uniform_op(const char* name, OpKind kind, const T* sendbuf, T* recvbuf, size_t count, ReductionOperator op,
                int root, typename Backend::comm_type& comm, typename Backend::req_type* req, int algo = 0) {
  AL_API_SCOPE(name);
  api_enter<Backend, T>(name, comm);
  debug::check_rank(root, comm.size());
  if ((kind == OpKind::reduce || kind == OpKind::reduce_scatter) && !reduction_supported(dtype_of<T>(), op))
    throw_al_exception(name, ": operator ", reduction_name(op), " is not defined for ", dtype_name(dtype_of<T>()));
  Resolved r = resolve_uniform(kind, dtype_of<T>(), sendbuf, recvbuf, count, op, root, comm.rank(), comm.size());
  debug::check_resolved(r, r.send != nullptr, r.recv != nullptr, comm.rank(), comm.size());
  Backend::run(std::move(r), comm, req, algo);
}
template <typename Backend, typename T>
void vector_op(const char* name, OpKind kind, const T* sendbuf, T* recvbuf, std::vector<size_t> sc,
               std::vector<size_t> sd, std::vector<size_t> rc, std::vector<size_t> rd, ReductionOperator op, int root,
               typename Backend::comm_type& comm, typename Backend::req_type* req, int algo = 0) {
  AL_API_SCOPE(name);
  api_enter<Backend, T>(name, comm);
  debug::check_rank(root, comm.size());
  Resolved r = resolve_vector(kind, dtype_of<T>(), sendbuf, recvbuf, std::move(sc), std::move(sd), std::move(rc),
                              std::move(rd), op, root, comm.rank(), comm.size());
  debug::check_resolved(r, r.send != nullptr, r.recv != nullptr, comm.rank(), comm.size());
  Backend::run(std::move(r), comm, req, algo);
}
}  // namespace internal

#define AL_SUM ReductionOperator::sum

// ============================ Reduce =========================================
template <typename Backend, typename T>
void Reduce(const T* sendbuf, T* recvbuf, size_t count, ReductionOperator op, int root, typename Backend::comm_type& comm,
            typename Backend::reduce_algo_type algo = Backend::reduce_algo_type::automatic) {
  internal::uniform_op<Backend, T>("reduce", internal::OpKind::reduce, sendbuf, recvbuf, count, op, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Reduce(T* buffer, size_t count, ReductionOperator op, int root, typename Backend::comm_type& comm,
            typename Backend::reduce_algo_type algo = Backend::reduce_algo_type::automatic) {
  internal::uniform_op<Backend, T>("reduce", internal::OpKind::reduce, internal::IN_PLACE<T>(), buffer, count, op, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingReduce(const T* sendbuf, T* recvbuf, size_t count, ReductionOperator op, int root,
                       typename Backend::comm_type& comm, typename Backend::req_type& req,
                       typename Backend::reduce_algo_type algo = Backend::reduce_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-reduce", internal::OpKind::reduce, sendbuf, recvbuf, count, op, root, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingReduce(T* buffer, size_t count, ReductionOperator op, int root, typename Backend::comm_type& comm,
                       typename Backend::req_type& req,
                       typename Backend::reduce_algo_type algo = Backend::reduce_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-reduce", internal::OpKind::reduce, internal::IN_PLACE<T>(), buffer, count, op, root, comm, &req, (int)algo);
}

// ============================ Reduce_scatter ==================================
/** `count` is the length each rank receives; the send buffer holds count * size elements. */
template <typename Backend, typename T>
void Reduce_scatter(const T* sendbuf, T* recvbuf, size_t count, ReductionOperator op, typename Backend::comm_type& comm,
                    typename Backend::reduce_scatter_algo_type algo = Backend::reduce_scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("reduce_scatter", internal::OpKind::reduce_scatter, sendbuf, recvbuf, count, op, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Reduce_scatter(T* buffer, size_t count, ReductionOperator op, typename Backend::comm_type& comm,
                    typename Backend::reduce_scatter_algo_type algo = Backend::reduce_scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("reduce_scatter", internal::OpKind::reduce_scatter, internal::IN_PLACE<T>(), buffer, count, op, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingReduce_scatter(const T* sendbuf, T* recvbuf, size_t count, ReductionOperator op,
                               typename Backend::comm_type& comm, typename Backend::req_type& req,
                               typename Backend::reduce_scatter_algo_type algo = Backend::reduce_scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-reduce_scatter", internal::OpKind::reduce_scatter, sendbuf, recvbuf, count, op, 0, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingReduce_scatter(T* buffer, size_t count, ReductionOperator op, typename Backend::comm_type& comm,
                               typename Backend::req_type& req,
                               typename Backend::reduce_scatter_algo_type algo = Backend::reduce_scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-reduce_scatter", internal::OpKind::reduce_scatter, internal::IN_PLACE<T>(), buffer, count, op, 0, comm, &req, (int)algo);
}

// ============================ Reduce_scatterv =================================
template <typename Backend, typename T>
void Reduce_scatterv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, ReductionOperator op,
                     typename Backend::comm_type& comm,
                     typename Backend::reduce_scatterv_algo_type = Backend::reduce_scatterv_algo_type::automatic) {
  debug::check_vector_is_comm_sized(counts, comm.size());
  internal::vector_op<Backend, T>("reduce_scatterv", internal::OpKind::reduce_scatter, sendbuf, recvbuf, {}, {}, std::move(counts), {}, op, 0, comm, nullptr);
}
template <typename Backend, typename T>
void Reduce_scatterv(T* buffer, std::vector<size_t> counts, ReductionOperator op, typename Backend::comm_type& comm,
                     typename Backend::reduce_scatterv_algo_type = Backend::reduce_scatterv_algo_type::automatic) {
  debug::check_vector_is_comm_sized(counts, comm.size());
  internal::vector_op<Backend, T>("reduce_scatterv", internal::OpKind::reduce_scatter, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), {}, op, 0, comm, nullptr);
}
template <typename Backend, typename T>
void NonblockingReduce_scatterv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, ReductionOperator op,
                                typename Backend::comm_type& comm, typename Backend::req_type& req,
                                typename Backend::reduce_scatterv_algo_type = Backend::reduce_scatterv_algo_type::automatic) {
  debug::check_vector_is_comm_sized(counts, comm.size());
  internal::vector_op<Backend, T>("nonblocking-reduce_scatterv", internal::OpKind::reduce_scatter, sendbuf, recvbuf, {}, {}, std::move(counts), {}, op, 0, comm, &req);
}
template <typename Backend, typename T>
void NonblockingReduce_scatterv(T* buffer, std::vector<size_t> counts, ReductionOperator op,
                                typename Backend::comm_type& comm, typename Backend::req_type& req,
                                typename Backend::reduce_scatterv_algo_type = Backend::reduce_scatterv_algo_type::automatic) {
  debug::check_vector_is_comm_sized(counts, comm.size());
  internal::vector_op<Backend, T>("nonblocking-reduce_scatterv", internal::OpKind::reduce_scatter, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), {}, op, 0, comm, &req);
}

// ============================ Allgather =======================================
/** `count` is each rank's contribution; the receive buffer holds count * size elements. */
template <typename Backend, typename T>
void Allgather(const T* sendbuf, T* recvbuf, size_t count, typename Backend::comm_type& comm,
               typename Backend::allgather_algo_type algo = Backend::allgather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("allgather", internal::OpKind::allgather, sendbuf, recvbuf, count, AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Allgather(T* buffer, size_t count, typename Backend::comm_type& comm,
               typename Backend::allgather_algo_type algo = Backend::allgather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("allgather", internal::OpKind::allgather, internal::IN_PLACE<T>(), buffer, count, AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAllgather(const T* sendbuf, T* recvbuf, size_t count, typename Backend::comm_type& comm,
                          typename Backend::req_type& req,
                          typename Backend::allgather_algo_type algo = Backend::allgather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-allgather", internal::OpKind::allgather, sendbuf, recvbuf, count, AL_SUM, 0, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAllgather(T* buffer, size_t count, typename Backend::comm_type& comm, typename Backend::req_type& req,
                          typename Backend::allgather_algo_type algo = Backend::allgather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-allgather", internal::OpKind::allgather, internal::IN_PLACE<T>(), buffer, count, AL_SUM, 0, comm, &req, (int)algo);
}

// ============================ Allgatherv ======================================
template <typename Backend, typename T>
void Allgatherv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, std::vector<size_t> displs,
                typename Backend::comm_type& comm,
                typename Backend::allgatherv_algo_type algo = Backend::allgatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("allgatherv", internal::OpKind::allgather, sendbuf, recvbuf, {}, {}, std::move(counts), std::move(displs), AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Allgatherv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs, typename Backend::comm_type& comm,
                typename Backend::allgatherv_algo_type algo = Backend::allgatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("allgatherv", internal::OpKind::allgather, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), std::move(displs), AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAllgatherv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, std::vector<size_t> displs,
                           typename Backend::comm_type& comm, typename Backend::req_type& req,
                           typename Backend::allgatherv_algo_type algo = Backend::allgatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-allgatherv", internal::OpKind::allgather, sendbuf, recvbuf, {}, {}, std::move(counts), std::move(displs), AL_SUM, 0, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAllgatherv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs,
                           typename Backend::comm_type& comm, typename Backend::req_type& req,
                           typename Backend::allgatherv_algo_type algo = Backend::allgatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-allgatherv", internal::OpKind::allgather, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), std::move(displs), AL_SUM, 0, comm, &req, (int)algo);
}

// ============================ Barrier =========================================
/** On the GPU backends a barrier synchronises the communicators' streams, not the hosts. */
template <typename Backend>
void Barrier(typename Backend::comm_type& comm,
             typename Backend::barrier_algo_type = Backend::barrier_algo_type::automatic) {
  AL_API_SCOPE("barrier");
  if (trace::enabled()) trace::record_op(Backend::Name().c_str(), DType::u8, "barrier", comm.rank(), comm.size());
  internal::Resolved r;
  Backend::run(std::move(r), comm, nullptr);
}
template <typename Backend>
void NonblockingBarrier(typename Backend::comm_type& comm, typename Backend::req_type& req,
                        typename Backend::barrier_algo_type = Backend::barrier_algo_type::automatic) {
  AL_API_SCOPE("nonblocking-barrier");
  if (trace::enabled()) trace::record_op(Backend::Name().c_str(), DType::u8, "nonblocking-barrier", comm.rank(), comm.size());
  internal::Resolved r;
  Backend::run(std::move(r), comm, &req);
}

// ============================ Bcast ===========================================
template <typename Backend, typename T>
void Bcast(T* buffer, size_t count, int root, typename Backend::comm_type& comm,
           typename Backend::bcast_algo_type algo = Backend::bcast_algo_type::automatic) {
  internal::uniform_op<Backend, T>("bcast", internal::OpKind::bcast, internal::IN_PLACE<T>(), buffer, count, AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingBcast(T* buffer, size_t count, int root, typename Backend::comm_type& comm,
                      typename Backend::req_type& req,
                      typename Backend::bcast_algo_type algo = Backend::bcast_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-bcast", internal::OpKind::bcast, internal::IN_PLACE<T>(), buffer, count, AL_SUM, root, comm, &req, (int)algo);
}

// ============================ Alltoall ========================================
/** `count` is the length of the slice exchanged with each peer. */
template <typename Backend, typename T>
void Alltoall(const T* sendbuf, T* recvbuf, size_t count, typename Backend::comm_type& comm,
              typename Backend::alltoall_algo_type algo = Backend::alltoall_algo_type::automatic) {
  internal::uniform_op<Backend, T>("alltoall", internal::OpKind::alltoall, sendbuf, recvbuf, count, AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Alltoall(T* buffer, size_t count, typename Backend::comm_type& comm,
              typename Backend::alltoall_algo_type algo = Backend::alltoall_algo_type::automatic) {
  internal::uniform_op<Backend, T>("alltoall", internal::OpKind::alltoall, internal::IN_PLACE<T>(), buffer, count, AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAlltoall(const T* sendbuf, T* recvbuf, size_t count, typename Backend::comm_type& comm,
                         typename Backend::req_type& req,
                         typename Backend::alltoall_algo_type algo = Backend::alltoall_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-alltoall", internal::OpKind::alltoall, sendbuf, recvbuf, count, AL_SUM, 0, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAlltoall(T* buffer, size_t count, typename Backend::comm_type& comm, typename Backend::req_type& req,
                         typename Backend::alltoall_algo_type algo = Backend::alltoall_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-alltoall", internal::OpKind::alltoall, internal::IN_PLACE<T>(), buffer, count, AL_SUM, 0, comm, &req, (int)algo);
}

// ============================ Alltoallv =======================================
template <typename Backend, typename T>
void Alltoallv(const T* sendbuf, std::vector<size_t> send_counts, std::vector<size_t> send_displs, T* recvbuf,
               std::vector<size_t> recv_counts, std::vector<size_t> recv_displs, typename Backend::comm_type& comm,
               typename Backend::alltoallv_algo_type algo = Backend::alltoallv_algo_type::automatic) {
  internal::vector_op<Backend, T>("alltoallv", internal::OpKind::alltoall, sendbuf, recvbuf, std::move(send_counts), std::move(send_displs), std::move(recv_counts), std::move(recv_displs), AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Alltoallv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs, typename Backend::comm_type& comm,
               typename Backend::alltoallv_algo_type algo = Backend::alltoallv_algo_type::automatic) {
  internal::vector_op<Backend, T>("alltoallv", internal::OpKind::alltoall, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), std::move(displs), AL_SUM, 0, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAlltoallv(const T* sendbuf, std::vector<size_t> send_counts, std::vector<size_t> send_displs,
                          T* recvbuf, std::vector<size_t> recv_counts, std::vector<size_t> recv_displs,
                          typename Backend::comm_type& comm, typename Backend::req_type& req,
                          typename Backend::alltoallv_algo_type algo = Backend::alltoallv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-alltoallv", internal::OpKind::alltoall, sendbuf, recvbuf, std::move(send_counts), std::move(send_displs), std::move(recv_counts), std::move(recv_displs), AL_SUM, 0, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingAlltoallv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs,
                          typename Backend::comm_type& comm, typename Backend::req_type& req,
                          typename Backend::alltoallv_algo_type algo = Backend::alltoallv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-alltoallv", internal::OpKind::alltoall, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), std::move(displs), AL_SUM, 0, comm, &req, (int)algo);
}

// ============================ Gather / Gatherv ================================
template <typename Backend, typename T>
void Gather(const T* sendbuf, T* recvbuf, size_t count, int root, typename Backend::comm_type& comm,
            typename Backend::gather_algo_type algo = Backend::gather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("gather", internal::OpKind::gather, sendbuf, recvbuf, count, AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Gather(T* buffer, size_t count, int root, typename Backend::comm_type& comm,
            typename Backend::gather_algo_type algo = Backend::gather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("gather", internal::OpKind::gather, internal::IN_PLACE<T>(), buffer, count, AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingGather(const T* sendbuf, T* recvbuf, size_t count, int root, typename Backend::comm_type& comm,
                       typename Backend::req_type& req,
                       typename Backend::gather_algo_type algo = Backend::gather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-gather", internal::OpKind::gather, sendbuf, recvbuf, count, AL_SUM, root, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingGather(T* buffer, size_t count, int root, typename Backend::comm_type& comm,
                       typename Backend::req_type& req,
                       typename Backend::gather_algo_type algo = Backend::gather_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-gather", internal::OpKind::gather, internal::IN_PLACE<T>(), buffer, count, AL_SUM, root, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void Gatherv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, std::vector<size_t> displs, int root,
             typename Backend::comm_type& comm,
             typename Backend::gatherv_algo_type algo = Backend::gatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("gatherv", internal::OpKind::gather, sendbuf, recvbuf, {}, {}, std::move(counts), std::move(displs), AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Gatherv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs, int root,
             typename Backend::comm_type& comm,
             typename Backend::gatherv_algo_type algo = Backend::gatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("gatherv", internal::OpKind::gather, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), std::move(displs), AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingGatherv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, std::vector<size_t> displs, int root,
                        typename Backend::comm_type& comm, typename Backend::req_type& req,
                        typename Backend::gatherv_algo_type algo = Backend::gatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-gatherv", internal::OpKind::gather, sendbuf, recvbuf, {}, {}, std::move(counts), std::move(displs), AL_SUM, root, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingGatherv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs, int root,
                        typename Backend::comm_type& comm, typename Backend::req_type& req,
                        typename Backend::gatherv_algo_type algo = Backend::gatherv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-gatherv", internal::OpKind::gather, internal::IN_PLACE<T>(), buffer, {}, {}, std::move(counts), std::move(displs), AL_SUM, root, comm, &req, (int)algo);
}

// ============================ Scatter / Scatterv ==============================
template <typename Backend, typename T>
void Scatter(const T* sendbuf, T* recvbuf, size_t count, int root, typename Backend::comm_type& comm,
             typename Backend::scatter_algo_type algo = Backend::scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("scatter", internal::OpKind::scatter, sendbuf, recvbuf, count, AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Scatter(T* buffer, size_t count, int root, typename Backend::comm_type& comm,
             typename Backend::scatter_algo_type algo = Backend::scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("scatter", internal::OpKind::scatter, internal::IN_PLACE<T>(), buffer, count, AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingScatter(const T* sendbuf, T* recvbuf, size_t count, int root, typename Backend::comm_type& comm,
                        typename Backend::req_type& req,
                        typename Backend::scatter_algo_type algo = Backend::scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-scatter", internal::OpKind::scatter, sendbuf, recvbuf, count, AL_SUM, root, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingScatter(T* buffer, size_t count, int root, typename Backend::comm_type& comm,
                        typename Backend::req_type& req,
                        typename Backend::scatter_algo_type algo = Backend::scatter_algo_type::automatic) {
  internal::uniform_op<Backend, T>("nonblocking-scatter", internal::OpKind::scatter, internal::IN_PLACE<T>(), buffer, count, AL_SUM, root, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void Scatterv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, std::vector<size_t> displs, int root,
              typename Backend::comm_type& comm,
              typename Backend::scatterv_algo_type algo = Backend::scatterv_algo_type::automatic) {
  internal::vector_op<Backend, T>("scatterv", internal::OpKind::scatter, sendbuf, recvbuf, std::move(counts), std::move(displs), {}, {}, AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void Scatterv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs, int root,
              typename Backend::comm_type& comm,
              typename Backend::scatterv_algo_type algo = Backend::scatterv_algo_type::automatic) {
  internal::vector_op<Backend, T>("scatterv", internal::OpKind::scatter, internal::IN_PLACE<T>(), buffer, std::move(counts), std::move(displs), {}, {}, AL_SUM, root, comm, nullptr, (int)algo);
}
template <typename Backend, typename T>
void NonblockingScatterv(const T* sendbuf, T* recvbuf, std::vector<size_t> counts, std::vector<size_t> displs,
                         int root, typename Backend::comm_type& comm, typename Backend::req_type& req,
                         typename Backend::scatterv_algo_type algo = Backend::scatterv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-scatterv", internal::OpKind::scatter, sendbuf, recvbuf, std::move(counts), std::move(displs), {}, {}, AL_SUM, root, comm, &req, (int)algo);
}
template <typename Backend, typename T>
void NonblockingScatterv(T* buffer, std::vector<size_t> counts, std::vector<size_t> displs, int root,
                         typename Backend::comm_type& comm, typename Backend::req_type& req,
                         typename Backend::scatterv_algo_type algo = Backend::scatterv_algo_type::automatic) {
  internal::vector_op<Backend, T>("nonblocking-scatterv", internal::OpKind::scatter, internal::IN_PLACE<T>(), buffer, std::move(counts), std::move(displs), {}, {}, AL_SUM, root, comm, &req, (int)algo);
}

// ============================ point-to-point ==================================
namespace internal {
template <typename Backend, typename T>
void p2p_op(const char* name, std::vector<typename Backend::p2p_item>&& items, typename Backend::comm_type& comm,
            typename Backend::req_type* req) {
  AL_API_SCOPE(name);
  api_enter<Backend, T>(name, comm);
  Backend::run_p2p(std::move(items), comm, req, name);
}
}  // namespace internal

/** Untagged send; matched in order with the receives `dest` posts for this rank. */
template <typename Backend, typename T>
void Send(const T* sendbuf, size_t count, int dest, typename Backend::comm_type& comm) {
  debug::check_rank(dest, comm.size());
  internal::p2p_op<Backend, T>("send", {Backend::make_send(sendbuf, count * sizeof(T), dest)}, comm, nullptr);
}
template <typename Backend, typename T>
void NonblockingSend(const T* sendbuf, size_t count, int dest, typename Backend::comm_type& comm,
                     typename Backend::req_type& req) {
  debug::check_rank(dest, comm.size());
  internal::p2p_op<Backend, T>("nonblocking-send", {Backend::make_send(sendbuf, count * sizeof(T), dest)}, comm, &req);
}
template <typename Backend, typename T>
void Recv(T* recvbuf, size_t count, int src, typename Backend::comm_type& comm) {
  debug::check_rank(src, comm.size());
  internal::p2p_op<Backend, T>("recv", {Backend::make_recv(recvbuf, count * sizeof(T), src)}, comm, nullptr);
}
template <typename Backend, typename T>
void NonblockingRecv(T* recvbuf, size_t count, int src, typename Backend::comm_type& comm,
                     typename Backend::req_type& req) {
  debug::check_rank(src, comm.size());
  internal::p2p_op<Backend, T>("nonblocking-recv", {Backend::make_recv(recvbuf, count * sizeof(T), src)}, comm, &req);
}
/** Send to `dest` and receive from `src` as one operation (they may differ). */
template <typename Backend, typename T>
void SendRecv(const T* sendbuf, size_t send_count, int dest, T* recvbuf, size_t recv_count, int src,
              typename Backend::comm_type& comm) {
  internal::p2p_op<Backend, T>("sendrecv", {Backend::make_send(sendbuf, send_count * sizeof(T), dest),
                                            Backend::make_recv(recvbuf, recv_count * sizeof(T), src)}, comm, nullptr);
}
/** In-place: `buffer` is sent to `dest`, then overwritten with `count` elements from `src`. */
template <typename Backend, typename T>
void SendRecv(T* buffer, size_t count, int dest, int src, typename Backend::comm_type& comm) {
  internal::p2p_op<Backend, T>("sendrecv", {Backend::make_send(buffer, count * sizeof(T), dest),
                                            Backend::make_recv(buffer, count * sizeof(T), src)}, comm, nullptr);
}
template <typename Backend, typename T>
void NonblockingSendRecv(const T* sendbuf, size_t send_count, int dest, T* recvbuf, size_t recv_count, int src,
                         typename Backend::comm_type& comm, typename Backend::req_type& req) {
  internal::p2p_op<Backend, T>("nonblocking-sendrecv", {Backend::make_send(sendbuf, send_count * sizeof(T), dest),
                                                        Backend::make_recv(recvbuf, recv_count * sizeof(T), src)}, comm, &req);
}
template <typename Backend, typename T>
void NonblockingSendRecv(T* buffer, size_t count, int dest, int src, typename Backend::comm_type& comm,
                         typename Backend::req_type& req) {
  internal::p2p_op<Backend, T>("nonblocking-sendrecv", {Backend::make_send(buffer, count * sizeof(T), dest),
                                                        Backend::make_recv(buffer, count * sizeof(T), src)}, comm, &req);
}

namespace internal {
template <typename Backend, typename T>
std::vector<typename Backend::p2p_item> multi_items(std::vector<const T*>& sbufs, std::vector<size_t>& scounts,
                                                    std::vector<int>& dests, std::vector<T*>& rbufs,
                                                    std::vector<size_t>& rcounts, std::vector<int>& srcs) {
  debug::check_multisendrecv(sbufs.size(), scounts.size(), dests.size(), rbufs.size(), rcounts.size(), srcs.size());
  std::vector<typename Backend::p2p_item> items;
  for (size_t i = 0; i < sbufs.size(); ++i) items.push_back(Backend::make_send(sbufs[i], scounts[i] * sizeof(T), dests[i]));
  for (size_t i = 0; i < rbufs.size(); ++i) items.push_back(Backend::make_recv(rbufs[i], rcounts[i] * sizeof(T), srcs[i]));
  return items;
}
}  // namespace internal

/** An arbitrary set of sends and receives that progress together as one operation. */
template <typename Backend, typename T>
void MultiSendRecv(std::vector<const T*> send_buffers, std::vector<size_t> send_counts, std::vector<int> dests,
                   std::vector<T*> recv_buffers, std::vector<size_t> recv_counts, std::vector<int> srcs,
                   typename Backend::comm_type& comm) {
  internal::p2p_op<Backend, T>("multisendrecv", internal::multi_items<Backend, T>(send_buffers, send_counts, dests, recv_buffers, recv_counts, srcs), comm, nullptr);
}
/** In-place: buffer i is sent to dests[i] and then overwritten from srcs[i]. */
template <typename Backend, typename T>
void MultiSendRecv(std::vector<T*> buffers, std::vector<size_t> counts, std::vector<int> dests, std::vector<int> srcs,
                   typename Backend::comm_type& comm) {
  std::vector<const T*> sb(buffers.begin(), buffers.end());
  internal::p2p_op<Backend, T>("multisendrecv", internal::multi_items<Backend, T>(sb, counts, dests, buffers, counts, srcs), comm, nullptr);
}
template <typename Backend, typename T>
void NonblockingMultiSendRecv(std::vector<const T*> send_buffers, std::vector<size_t> send_counts,
                              std::vector<int> dests, std::vector<T*> recv_buffers, std::vector<size_t> recv_counts,
                              std::vector<int> srcs, typename Backend::comm_type& comm,
                              typename Backend::req_type& req) {
  internal::p2p_op<Backend, T>("nonblocking-multisendrecv", internal::multi_items<Backend, T>(send_buffers, send_counts, dests, recv_buffers, recv_counts, srcs), comm, &req);
}
template <typename Backend, typename T>
void NonblockingMultiSendRecv(std::vector<T*> buffers, std::vector<size_t> counts, std::vector<int> dests,
                              std::vector<int> srcs, typename Backend::comm_type& comm,
                              typename Backend::req_type& req) {
  std::vector<const T*> sb(buffers.begin(), buffers.end());
  internal::p2p_op<Backend, T>("nonblocking-multisendrecv", internal::multi_items<Backend, T>(sb, counts, dests, buffers, counts, srcs), comm, &req);
}

// ============================ completion ======================================
/** Host-side poll. Returns true once the operation has completed and resets `req` to null. */
template <typename Backend>
bool Test(typename Backend::req_type& req) { return Backend::test(req); }
/**
 * Wait for a non-blocking operation.  Host backend: blocks the caller.  GPU
 * backends: makes the communicator's stream wait; the host returns at once.
 * `req` is null afterwards.
 */
template <typename Backend>
void Wait(typename Backend::req_type& req) { Backend::wait(req); }

// ============================ registration ====================================
template <typename Backend, typename T>
void RegisterMemory(T* buffer, size_t count, typename Backend::comm_type& comm) {
  Backend::register_memory(buffer, count * sizeof(T), comm);
}
template <typename Backend, typename T>
void UnregisterMemory(T* buffer, typename Backend::comm_type& comm) {
  Backend::unregister_memory(buffer, comm);
}

#undef AL_SUM
#undef AL_API_ENTER
}  // namespace Al

// Source compatibility with code written against the reference's backend names.
#ifndef AL_NO_REFERENCE_ALIASES
namespace Al {
using MPIBackend = HostBackend;
#ifdef AL_HAS_CUDA
using NCCLBackend = DeviceBackend;
#endif
}  // namespace Al
#endif
