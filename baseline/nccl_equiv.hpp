// Baseline only: the NCCL call sequences the reference's NCCL backend issues for
// each operation (include/aluminum/nccl_impl.hpp:944-1399 of the reference),
// reproduced call for call so that "the reference's NCCL backend" can be timed on
// the same box without MPI.  Nothing in the library proper uses this file.
//
//   allreduce       ncclAllReduce                                  (nccl_impl.hpp:951)
//   reduce_scatter  ncclReduceScatter                              (:1306)
//   allgather       ncclAllGather                                  (:1193)
//   alltoall        one group of p x (ncclSend + ncclRecv)         (:1235-1244)
//   bcast           ncclBroadcast                                  (:1096)
//   reduce          ncclReduce                                     (:1180)
//   sendrecv        grouped ncclSend + ncclRecv                    (:993-1006)
//
// NCCL is loaded with dlopen so that the tools still build and start where it is
// absent; the communicator is bootstrapped like the reference does (rank 0 creates
// the unique id, it is broadcast - here over the library's control plane instead
// of MPI - and every rank calls ncclCommInitRank, src/nccl_impl.cpp:52-59).
#pragma once
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "al/bootstrap.hpp"

namespace nccl_equiv {

struct UniqueId { char internal[128]; };
using Comm = void*;
enum DataType { Int8 = 0, Uint8 = 1, Int32 = 2, Uint32 = 3, Int64 = 4, Uint64 = 5, Float16 = 6, Float32 = 7, Float64 = 8, Bfloat16 = 9 };
enum RedOp { Sum = 0, Prod = 1, Max = 2, Min = 3, Avg = 4 };

struct Api {
  int (*GetUniqueId)(UniqueId*) = nullptr;
  int (*CommInitRank)(Comm*, int, UniqueId, int) = nullptr;
  int (*CommDestroy)(Comm) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*ReduceScatter)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, Comm, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Reduce)(const void*, void*, size_t, int, int, int, Comm, cudaStream_t) = nullptr;
  int (*Send)(const void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*Recv)(void*, size_t, int, int, Comm, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  // user-buffer registration, as Al::RegisterMemory<NCCLBackend> does (src/nccl_impl.cpp:83-109): optional symbols
  int (*MemAlloc)(void**, size_t) = nullptr;
  int (*MemFree)(void*) = nullptr;
  int (*CommRegister)(Comm, void*, size_t, void**) = nullptr;
  int (*CommDeregister)(Comm, void*) = nullptr;
  bool ok = false;
};

inline Api& api() {
  static Api a = [] {
    Api x;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return x;
#define L(field, sym) x.field = (decltype(x.field))dlsym(h, sym)
    L(GetUniqueId, "ncclGetUniqueId"); L(CommInitRank, "ncclCommInitRank"); L(CommDestroy, "ncclCommDestroy");
    L(AllReduce, "ncclAllReduce"); L(ReduceScatter, "ncclReduceScatter"); L(AllGather, "ncclAllGather");
    L(Broadcast, "ncclBroadcast"); L(Reduce, "ncclReduce"); L(Send, "ncclSend"); L(Recv, "ncclRecv");
    L(GroupStart, "ncclGroupStart"); L(GroupEnd, "ncclGroupEnd"); L(GetErrorString, "ncclGetErrorString");
    L(MemAlloc, "ncclMemAlloc"); L(MemFree, "ncclMemFree"); L(CommRegister, "ncclCommRegister"); L(CommDeregister, "ncclCommDeregister");
#undef L
    x.ok = x.GetUniqueId && x.CommInitRank && x.AllReduce && x.ReduceScatter && x.AllGather && x.Send && x.Recv &&
           x.GroupStart && x.GroupEnd;
    return x;
  }();
  return a;
}

inline void check(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string("NCCL error in ") + what + ": " +
                                        (api().GetErrorString ? api().GetErrorString(rc) : std::to_string(rc)));
}

class Communicator {
 public:
  Communicator(const Al::internal::Group& g, cudaStream_t stream) : rank_(g.rank()), size_(g.size()), stream_(stream) {
    if (!api().ok) throw std::runtime_error("libnccl could not be loaded");
    UniqueId id{};
    if (rank_ == 0) check(api().GetUniqueId(&id), "ncclGetUniqueId");
    g.bcast(&id, sizeof(id), 0);
    check(api().CommInitRank(&comm_, size_, id, rank_), "ncclCommInitRank");
  }
  ~Communicator() { if (comm_ && api().CommDestroy) api().CommDestroy(comm_); }
  int rank() const { return rank_; }
  int size() const { return size_; }
  cudaStream_t stream() const { return stream_; }

  /**
   * Memory that NCCL can use without its own staging copies: ncclMemAlloc + ncclCommRegister, the registered
   * counterpart of this library's symm_alloc / RegisterMemory (what a user of the reference gets from
   * Al::RegisterMemory<NCCLBackend> on an ncclMemAlloc'ed buffer).  nullptr when this NCCL lacks the calls.
   */
  void* alloc_registered(size_t bytes) {
    if (!api().MemAlloc || !api().CommRegister) return nullptr;
    void* p = nullptr;
    check(api().MemAlloc(&p, bytes), "ncclMemAlloc");
    void* handle = nullptr;
    check(api().CommRegister(comm_, p, bytes, &handle), "ncclCommRegister");
    registered_.push_back({p, handle});
    return p;
  }
  void free_registered(void* p) {
    for (auto it = registered_.begin(); it != registered_.end(); ++it) {
      if (it->first != p) continue;
      if (api().CommDeregister) check(api().CommDeregister(comm_, it->second), "ncclCommDeregister");
      if (api().MemFree) check(api().MemFree(p), "ncclMemFree");
      registered_.erase(it);
      return;
    }
  }

  void allreduce(const void* s, void* r, size_t n, int dt, int op) { check(api().AllReduce(s, r, n, dt, op, comm_, stream_), "ncclAllReduce"); }
  void reduce_scatter(const void* s, void* r, size_t n, int dt, int op) { check(api().ReduceScatter(s, r, n, dt, op, comm_, stream_), "ncclReduceScatter"); }
  void allgather(const void* s, void* r, size_t n, int dt) { check(api().AllGather(s, r, n, dt, comm_, stream_), "ncclAllGather"); }
  void bcast(void* b, size_t n, int dt, int root) { check(api().Broadcast(b, b, n, dt, root, comm_, stream_), "ncclBroadcast"); }
  void reduce(const void* s, void* r, size_t n, int dt, int op, int root) { check(api().Reduce(s, r, n, dt, op, root, comm_, stream_), "ncclReduce"); }
  /** p x (send + recv) in one group, self included, as the reference does. */
  void alltoall(const void* s, void* r, size_t n, int dt, size_t esz) {
    check(api().GroupStart(), "ncclGroupStart");
    for (int i = 0; i < size_; ++i) {
      check(api().Send((const char*)s + (size_t)i * n * esz, n, dt, i, comm_, stream_), "ncclSend");
      check(api().Recv((char*)r + (size_t)i * n * esz, n, dt, i, comm_, stream_), "ncclRecv");
    }
    check(api().GroupEnd(), "ncclGroupEnd");
  }
  void sendrecv(const void* s, size_t ns, int dest, void* r, size_t nr, int src, int dt) {
    check(api().GroupStart(), "ncclGroupStart");
    check(api().Send(s, ns, dt, dest, comm_, stream_), "ncclSend");
    check(api().Recv(r, nr, dt, src, comm_, stream_), "ncclRecv");
    check(api().GroupEnd(), "ncclGroupEnd");
  }

 private:
  int rank_, size_;
  cudaStream_t stream_;
  Comm comm_ = nullptr;
  std::vector<std::pair<void*, void*>> registered_;
};

}  // namespace nccl_equiv
