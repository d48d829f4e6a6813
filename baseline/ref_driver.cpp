// C interface over the UNMODIFIED reference library (llnl/Aluminum built by
// baseline/build_reference.py), for ctypes.  Every function below is a direct call of the
// reference's public API with its NCCL backend - Al::Initialize, Al::NCCLBackend::comm_type,
// Al::NonblockingAllreduce + Al::Wait, Al::Allreduce, Al::Reduce_scatter, Al::Allgather,
// Al::Alltoall (include/Al.hpp and include/aluminum/nccl_impl.hpp of the reference).  Nothing of the
// aluminum-b200 library is included or linked here: this file only exists so that the baseline
// can be driven from the same Python benchmark as the product.
#include <Al.hpp>

#include <cuda_runtime.h>

#include <cstdio>
#include <cstring>
#include <string>

namespace {
std::string g_err;
using B = Al::NCCLBackend;

template <typename F>
int guarded(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown exception";
    return 1;
  }
}

Al::ReductionOperator op_of(int op) {
  switch (op) {
    case 0: return Al::ReductionOperator::sum;
    case 1: return Al::ReductionOperator::prod;
    case 2: return Al::ReductionOperator::min;
    case 3: return Al::ReductionOperator::max;
    default: return Al::ReductionOperator::avg;
  }
}

struct Req {
  B::req_type r = B::null_req;
};

// kind: 0 allreduce, 1 reduce_scatter, 2 allgather, 3 alltoall
template <typename T>
void collective(B::comm_type& comm, int kind, const void* send, void* recv, size_t count, int op) {
  const T* s = (const T*)send;
  T* r = (T*)recv;
  switch (kind) {
    case 0:
      if (s == r || s == nullptr) Al::Allreduce<B>(r, count, op_of(op), comm);
      else Al::Allreduce<B>(s, r, count, op_of(op), comm);
      break;
    case 1: Al::Reduce_scatter<B>(s, r, count, op_of(op), comm); break;
    case 2: Al::Allgather<B>(s, r, count, comm); break;
    case 3: Al::Alltoall<B>(s, r, count, comm); break;
    default: throw std::runtime_error("unknown collective kind");
  }
}
}  // namespace

extern "C" {

const char* refal_last_error() { return g_err.c_str(); }
const char* refal_version() { return AL_VERSION; }

/** cudaSetDevice(device) then Al::Initialize (MPI stand-in, progress engine, CUDA and NCCL set-up). */
int refal_init(int device) {
  return guarded([&] {
    if (cudaSetDevice(device) != cudaSuccess) throw std::runtime_error("cudaSetDevice failed");
    int argc = 0;
    char** argv = nullptr;
    Al::Initialize(argc, argv);
  });
}
int refal_finalize() { return guarded([] { Al::Finalize(); }); }

/** World NCCL communicator bound to `stream` (ncclCommInitRank happens here). */
void* refal_comm_create(void* stream) {
  B::comm_type* c = nullptr;
  if (guarded([&] { c = new B::comm_type(MPI_COMM_WORLD, (cudaStream_t)stream); })) return nullptr;
  return c;
}
void refal_comm_destroy(void* comm) { (void)guarded([&] { delete (B::comm_type*)comm; }); }
int refal_rank(void* comm) { return ((B::comm_type*)comm)->rank(); }
int refal_size(void* comm) { return ((B::comm_type*)comm)->size(); }

/** Al::NonblockingAllreduce<NCCLBackend> in place; dtype 0 = float, 1 = bf16.  Returns a request handle. */
void* refal_nb_allreduce(void* comm, void* buf, size_t count, int dtype, int op) {
  Req* q = new Req;
  const int rc = guarded([&] {
    B::comm_type& c = *(B::comm_type*)comm;
    if (dtype == 0) Al::NonblockingAllreduce<B>((float*)buf, count, op_of(op), c, q->r);
    else Al::NonblockingAllreduce<B>((al_bfloat16*)buf, count, op_of(op), c, q->r);
  });
  if (rc) { delete q; return nullptr; }
  return q;
}
/** Al::Wait<NCCLBackend>: the communicator's stream waits for the operation; the host does not. */
int refal_wait(void* req) {
  Req* q = (Req*)req;
  const int rc = guarded([&] { Al::Wait<B>(q->r); });
  delete q;
  return rc;
}

/** Blocking (stream-ordered) collective on the communicator's stream. */
int refal_collective(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op) {
  return guarded([&] {
    B::comm_type& c = *(B::comm_type*)comm;
    if (dtype == 0) collective<float>(c, kind, send, recv, count, op);
    else collective<al_bfloat16>(c, kind, send, recv, count, op);
  });
}

/**
 * `warmup` untimed then `iters` timed calls, each preceded by MPI_Barrier and bracketed by a CUDA event
 * pair on the communicator's stream: the protocol of the reference's own benchmark
 * (benchmark/benchmark_ops.cpp:184-191, benchmark/benchmark_utils_nccl.hpp:46-58).
 */
int refal_time_collective(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op,
                          int warmup, int iters, float* out_ms) {
  return guarded([&] {
    B::comm_type& c = *(B::comm_type*)comm;
    cudaStream_t s = c.get_stream();
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess)
      throw std::runtime_error("cudaEventCreate failed");
    // The reference's benchmark lines the ranks up on MPI_COMM_WORLD (benchmark/benchmark_ops.cpp:185).
    int world = 0;
    MPI_Comm_size(MPI_COMM_WORLD, &world);
    MPI_Comm start_line = c.size() == world ? MPI_COMM_WORLD : c.get_comm();
    for (int i = 0; i < warmup + iters; ++i) {
      MPI_Barrier(start_line);
      cudaEventRecord(e0, s);
      if (dtype == 0) collective<float>(c, kind, send, recv, count, op);
      else collective<al_bfloat16>(c, kind, send, recv, count, op);
      cudaEventRecord(e1, s);
      if (cudaEventSynchronize(e1) != cudaSuccess) throw std::runtime_error("cudaEventSynchronize failed");
      float ms = 0;
      cudaEventElapsedTime(&ms, e0, e1);
      if (i >= warmup) out_ms[i - warmup] = ms;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
  });
}

/** Host-side helpers over the communicator's MPI communicator (timing: barrier, max over ranks). */
int refal_host_barrier(void* comm) {
  return guarded([&] { MPI_Barrier(((B::comm_type*)comm)->get_comm()); });
}
double refal_host_max(void* comm, double v) {
  double out = v;
  (void)guarded([&] { MPI_Allreduce(&v, &out, 1, MPI_DOUBLE, MPI_MAX, ((B::comm_type*)comm)->get_comm()); });
  return out;
}
int refal_host_bcast(void* comm, void* buf, int nbytes, int root) {
  return guarded([&] { MPI_Bcast(buf, nbytes, MPI_BYTE, root, ((B::comm_type*)comm)->get_comm()); });
}

}  // extern "C"
