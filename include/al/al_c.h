/**
 * @file al_c.h
 * C interface of the library (used by the Python package through ctypes).
 *
 * Every function returns 0 on success and non-zero on failure unless stated
 * otherwise; al_last_error() then describes the failure (thread-local).
 * Datatype, operator and collective codes are the numeric values of
 * Al::DType, Al::ReductionOperator and Al::internal::OpKind.
 * Buffers are raw addresses: host memory for the host backend, device memory
 * for the device backend.  `stream` arguments are cudaStream_t handles; pass
 * AL_C_COMM_STREAM to use the stream the communicator was created with.
 */
#pragma once
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AL_C_COMM_STREAM ((void*)(intptr_t)-1)

const char* al_last_error(void);
int al_init(void);
int al_finalize(void);
int al_initialized(void);
int al_world_rank(void);
int al_world_size(void);
int al_world_local_rank(void);
int al_world_local_size(void);
/** 1 while the process of `world_rank` still holds its control connection, 0 once it has exited or finalised, -1 on error. */
int al_world_peer_alive(int world_rank);
/** Number of nodes the world spans, and the index of this rank's node (0-based, by lowest rank). */
int al_world_num_nodes(void);
int al_world_node_index(void);
int al_cuda_available(void);
/** Writes a NUL-terminated description (version, features, tuning, topology) into buf. */
int al_info(char* buf, size_t buflen);
int al_set_tuning(const char* name, double value);
double al_get_tuning(const char* name);

/* ---- trace ---- */
void al_trace_enable(int on);
int al_trace_snapshot(char* buf, size_t buflen);
void al_trace_clear(void);

/* ---- host backend ---- */
void* al_host_comm_create(void);
/**
 * Communicator over the listed world ranks, in that order.  Collective over those ranks only
 * (every one of them passes the same list); the calling rank must be in it.
 */
void* al_host_comm_create_group(const int* world_ranks, int n);
void* al_host_comm_split(void* comm, int color, int key);
void al_host_comm_destroy(void* comm);
int al_host_comm_rank(void* comm);
int al_host_comm_size(void* comm);
/** Rank among / number of the communicator's members on this rank's node. */
int al_host_comm_local_rank(void* comm);
int al_host_comm_local_size(void* comm);
/** Collective: communicator of the members on this rank's node (NULL + al_last_error() on failure). */
void* al_host_comm_local(void* comm);
/** Fills out[0..3]: collectives, p2p_ops, bytes, failures. */
int al_host_comm_stats(void* comm, uint64_t* out);
/** Puts the communicator into the failed state on this rank (why may be NULL). */
int al_host_comm_abort(void* comm, const char* why);
/**
 * kind: OpKind.  inplace != 0 selects the in-place form on `recv`.
 * vector != 0 uses the count / displacement arrays (entries per rank; unused ones may be NULL).
 * req_out != NULL makes the call non-blocking and stores a request handle.
 */
int al_host_collective(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op, int root,
                       int inplace, int vector, const size_t* send_counts, const size_t* send_displs,
                       const size_t* recv_counts, const size_t* recv_displs, void** req_out);
/** n transfers: is_send[i], peer[i], buf[i], bytes[i]. */
int al_host_p2p(void* comm, int n, const int* is_send, const int* peer, void* const* buf, const size_t* bytes,
                void** req_out);
/** *done = 1 and the handle is released when complete. */
int al_host_test(void** req, int* done);
int al_host_wait(void** req);

/* ---- device backend ---- */
void* al_dev_comm_create(void* stream);
void* al_dev_comm_create_emulated(int p, void* stream);
/** As al_host_comm_create_group, for a device communicator on `stream`. */
void* al_dev_comm_create_group(const int* world_ranks, int n, void* stream);
void* al_dev_comm_split(void* comm, int color, int key, void* stream);
void al_dev_comm_destroy(void* comm);
int al_dev_comm_rank(void* comm);
int al_dev_comm_size(void* comm);
int al_dev_comm_nlocal(void* comm);
int al_dev_comm_has_multicast(void* comm);
const char* al_dev_comm_backing(void* comm);
int al_dev_comm_set_timeout_ms(void* comm, double ms);
/** Every later call on the communicator fails (why may be NULL). */
int al_dev_comm_abort(void* comm, const char* why);
/** Fills out[0..12]: ops, bytes, kernels, timeouts, one_shot, two_shot, nvls, nvls_zero_copy, bulk_pipeline, window, ll, rows, rs_nvls. */
int al_dev_comm_stats(void* comm, uint64_t* out);
/** Status record: out[0]=code, [1]=rank, [2]=peer, [3]=where, [4]=epoch, [5]=seen. Never fails. */
int al_dev_comm_status(void* comm, uint64_t* out);
/**
 * nlocal entries in send / recv (1 outside emulation).  Count tables, when
 * vector != 0, hold nlocal * size entries each (row per local rank).
 * dt_wire / dt_out < 0 mean "same as dt_in".  algo, for allreduce: 0 auto, 1 one-shot, 2 two-shot,
 * 3 NVLS, 4 low-latency packets; for every other collective it selects the data path: 0 auto, 1 staged,
 * 2 window (registered buffers), 3 low-latency packets.
 */
int al_dev_collective(void* comm, int kind, int nlocal, const void* const* send, void* const* recv, size_t count,
                      int dt_in, int dt_wire, int dt_out, int op, int root, int inplace, int vector,
                      const size_t* send_counts, const size_t* send_displs, const size_t* recv_counts,
                      const size_t* recv_displs, double scale, int algo, int ctas, void* stream, void** req_out);
/**
 * Alltoall(v) of strided or index-selected rows with the pack / unpack fused in.  Row k of what local rank lr
 * sends to peer d is read at send[lr] + send_peer_off[d] + id * send_row_stride with id = send_first[d] + k, or
 * send_idx[lr][send_first[d] + k] when an index array (device memory) is given; the receiving side mirrors it.
 * The six tables hold nlocal * size entries (a row per local rank); offsets and strides are in bytes.
 */
int al_dev_exchange_rows(void* comm, int nlocal, const void* const* send, void* const* recv, const long long* const* send_idx,
                         const long long* const* recv_idx, size_t row_bytes, size_t send_row_stride, size_t recv_row_stride,
                         const size_t* send_rows, const size_t* send_first, const size_t* send_peer_off,
                         const size_t* recv_rows, const size_t* recv_first, const size_t* recv_peer_off, void* stream,
                         void** req_out);
/**
 * Where the time of a small collective goes.  Same loop as al_dev_time_collective, with the kernels'
 * %globaltimer stamps switched on.  out_us[0..5] = medians in microseconds of: the event-pair time, the host
 * time inside the enqueueing call, kernel entry -> data sent, data sent -> first data seen, first data seen ->
 * kernel exit, kernel entry -> exit.  Event time minus kernel time is launch and front-end overhead.
 */
int al_dev_latency_breakdown(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op,
                             int algo, int warmup, int iters, void* stream, double* out_us);
/**
 * Collective over the communicator: make [ptr, ptr+bytes) of every rank addressable by all ranks (CUDA IPC for
 * cudaMalloc memory; symm_alloc memory is registered already).  Returns the window index (>= 0), -1 when some
 * rank's memory cannot be shared (nobody registers then; the buffer keeps using the staging path), -2 on error.
 */
int al_dev_register(void* comm, void* ptr, size_t bytes);
/** Emulated communicators: the n = size buffers of all ranks at once. */
int al_dev_register_emulated(void* comm, void* const* ptrs, int n, size_t bytes);
/** Collective: forget a registered buffer; call it before the memory is freed. */
int al_dev_unregister(void* comm, void* ptr);
/**
 * Benchmark helper: `warmup` untimed then `iters` timed out-of-place calls of one collective, each
 * preceded by a host barrier of the communicator's ranks and bracketed by a CUDA event pair on
 * `stream` (the reference's own timing protocol, benchmark/benchmark_ops.cpp:184-191).
 * out_ms receives the `iters` device times in milliseconds.
 */
int al_dev_time_collective(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op,
                           int warmup, int iters, void* stream, float* out_ms);
/** owner[i] is the issuing rank (emulation) or ignored. */
int al_dev_p2p(void* comm, int n, const int* is_send, const int* peer, const int* owner, void* const* buf,
               const size_t* bytes, void* stream, void** req_out);
int al_dev_test(void** req, int* done);
int al_dev_wait(void** req);
void* al_dev_symm_alloc(void* comm, size_t bytes);
int al_dev_symm_free(void* comm, void* ptr);
/** Guard mode (tuning entry debug_guard): fails if anything wrote outside a symm_alloc buffer of this rank. */
int al_dev_check_guards(void* comm);
/** Address of rank `peer`'s copy of the symmetric allocation that contains `local_ptr`. */
void* al_dev_symm_peer_ptr(void* comm, void* local_ptr, int peer);

/* ---- RMA / halo ---- */
void* al_rma_attach(void* comm, void* local_buf, int peer);
int al_rma_detach(void* comm, void* remote_buf, int peer);
int al_rma_put(void* comm, const void* src, int dest, void* dest_remote, size_t bytes);
/** Copy `bytes` out of `src_remote` (from al_rma_attach for rank src_rank) into local `dst`, stream-ordered. */
int al_rma_get(void* comm, void* dst, int src_rank, const void* src_remote, size_t bytes);
int al_rma_notify(void* comm, int peer);
int al_rma_wait(void* comm, int peer);
int al_rma_sync(void* comm, int peer);
/**
 * Fused halo exchange of a float tensor (nc, d_local + 2*depth, plane) split
 * along its second dimension.  tensors[r] is rank r's tensor as mapped in this
 * process (this rank's own tensor and those of its neighbours must be valid,
 * e.g. obtained with al_dev_symm_peer_ptr or al_rma_attach; in emulation all).
 * Ranks are chained in order: the neighbours of r are r-1 and r+1; with
 * periodic != 0 the chain is closed.
 */
int al_halo_exchange(void* comm, float* const* tensors, size_t nc, size_t d_local, size_t plane, size_t depth,
                     int periodic, int ctas, void* stream);
int al_halo_pack(float* packed, const float* tensor, size_t nc, size_t d_total, size_t plane, size_t d_first,
                 size_t depth, int unpack, void* stream);

/* ---- element-wise kernels ---- */
int al_scale_cast(void* out, int out_dt, const void* in, int in_dt, size_t n, double scale, void* stream);
int al_sgd_momentum(float* param, float* momentum, float* grad, size_t n, float lr, float mu, float weight_decay,
                    float grad_scale, int first_step, int zero_grad, void* stream);
int al_fill_u32(void* out, size_t n, uint32_t value, void* stream);

#ifdef __cplusplus
}
#endif
