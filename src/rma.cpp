// One-sided extension (see al/rma.hpp).
#include "al/rma.hpp"

#include <map>
#include <mutex>

#include "al/device/kernels.hpp"
#include "al/tuning.hpp"

namespace Al {
namespace internal {
namespace rma {

namespace {

struct AttachMsg {
  int kind;            // 0 null, 1 symmetric block, 2 cudaIpc handle
  int block_index;     // kind 1: index in the sender's list of symmetric blocks (same order on every rank)
  size_t offset;       // offset of the buffer inside the block / the IPC allocation
  cudaIpcMemHandle_t handle;
};

struct Opened { void* base; int refs; };

struct State {
  std::vector<uint64_t> notified, waited;                 // per peer
  std::map<std::pair<int, std::string>, Opened> opened;   // (peer, handle bytes) -> mapping
  std::map<void*, std::pair<int, std::string>> by_ptr;    // returned pointer -> key
};

// Never destroyed: communicators may outlive the static objects of this file at process exit.
std::mutex& g_mu = *new std::mutex;
std::map<const void*, State>& g_states = *new std::map<const void*, State>;

State& state_of(DeviceCommunicator& comm) {
  State& s = g_states[comm.impl()];
  if (s.notified.empty()) {
    s.notified.assign((size_t)comm.size(), 0);
    s.waited.assign((size_t)comm.size(), 0);
  }
  return s;
}

}  // namespace

void* attach(void* local_buf, int peer, DeviceCommunicator& comm) {
  if (peer < 0) return nullptr;                 // null connection
  if (peer == comm.rank() || comm.is_emulated()) return local_buf;  // self connection
  if (peer >= comm.size()) throw_al_exception("attach: peer ", peer, " out of range");
  std::lock_guard<std::mutex> g(g_mu);
  State& st = state_of(comm);
  AttachMsg mine{};
  size_t off = 0;
  const device::SymmBlock* sb = local_buf ? comm.find_symm(local_buf, 1, &off) : nullptr;
  if (!local_buf) {
    mine.kind = 0;
  } else if (sb) {
    mine.kind = 1;
    mine.offset = off;
    mine.block_index = comm.symm_index(local_buf);  // blocks are allocated collectively: same index on every rank
  } else {
    mine.kind = 2;
    CUdeviceptr base = 0;
    size_t size = 0;
    const auto& d = cuda::drv();
    if (!d.MemGetAddressRange || d.MemGetAddressRange(&base, &size, (CUdeviceptr)local_buf) != CUDA_SUCCESS)
      throw_al_exception("attach: cannot determine the allocation of the buffer");
    mine.offset = (size_t)((CUdeviceptr)local_buf - base);
    AL_CHECK_CUDA(cudaIpcGetMemHandle(&mine.handle, (void*)base));
  }
  AttachMsg out = mine, in{};
  World* w = comm.group().world();
  const int wpeer = comm.group().world_rank_of(peer);
  {
    std::lock_guard<std::mutex> cg(w->collective_mutex());
    if (comm.rank() < peer) { w->send(wpeer, &out, sizeof(out)); w->recv(wpeer, &in, sizeof(in)); }
    else { w->recv(wpeer, &in, sizeof(in)); w->send(wpeer, &out, sizeof(out)); }
  }
  if (in.kind == 0) return nullptr;
  if (in.kind == 1) {
    void* p = comm.symm_peer_ptr(in.block_index, peer, in.offset);
    if (!p) throw_al_exception("attach: peer's symmetric buffer is unknown to this rank");
    return p;
  }
  std::string key((const char*)&in.handle, sizeof(in.handle));
  auto k = std::make_pair(peer, key);
  auto it = st.opened.find(k);
  if (it == st.opened.end()) {
    void* base = nullptr;
    AL_CHECK_CUDA(cudaIpcOpenMemHandle(&base, in.handle, cudaIpcMemLazyEnablePeerAccess));
    it = st.opened.emplace(k, Opened{base, 0}).first;
  }
  it->second.refs++;
  void* ret = (char*)it->second.base + in.offset;
  st.by_ptr[ret] = k;
  return ret;
}

void detach(void* remote_buf, int peer, DeviceCommunicator& comm) {
  if (peer < 0 || !remote_buf || peer == comm.rank() || comm.is_emulated()) return;
  std::lock_guard<std::mutex> g(g_mu);
  State& st = state_of(comm);
  auto it = st.by_ptr.find(remote_buf);
  if (it == st.by_ptr.end()) return;  // symmetric memory: nothing to close
  auto oit = st.opened.find(it->second);
  st.by_ptr.erase(it);
  if (oit != st.opened.end() && --oit->second.refs == 0) {
    AL_CHECK_CUDA(cudaStreamSynchronize(comm.get_stream()));
    AL_WARN_CUDA(cudaIpcCloseMemHandle(oit->second.base));
    st.opened.erase(oit);
  }
}

void forget(const void* comm_impl) noexcept {
  // A later communicator may be allocated at the same address: it must start from zeroed counters,
  // like its flag area.
  try {
    std::lock_guard<std::mutex> g(g_mu);
    auto it = g_states.find(comm_impl);
    if (it == g_states.end()) return;
    for (auto& o : it->second.opened) AL_WARN_CUDA(cudaIpcCloseMemHandle(o.second.base));
    g_states.erase(it);
  } catch (...) {
  }
}

void notify(int peer, DeviceCommunicator& comm) {
  if (peer < 0) return;
  std::lock_guard<std::mutex> g(g_mu);
  State& st = state_of(comm);
  comm.check_status();
  const device::Workspace& ws = comm.workspace();
  const int me = comm.rank();
  uint64_t* word = ws.flags[peer] + device::FlagLayout::off_rma + (size_t)me * device::FlagLayout::stride;
  device::launch_signal(word, ++st.notified[(size_t)peer], comm.get_stream());
}

void wait(int peer, DeviceCommunicator& comm) {
  if (peer < 0) return;
  std::lock_guard<std::mutex> g(g_mu);
  State& st = state_of(comm);
  comm.check_status();
  const device::Workspace& ws = comm.workspace();
  const int me = comm.rank();
  const uint64_t* word = ws.flags[me] + device::FlagLayout::off_rma + (size_t)peer * device::FlagLayout::stride;
  device::launch_wait_word(word, ++st.waited[(size_t)peer], comm.wait_timeout_ns(), ws, me, peer, comm.get_stream());
}

void put(const void* src, int dest, void* dest_remote, size_t bytes, DeviceCommunicator& comm) {
  if (dest < 0 || bytes == 0) return;
  if (!dest_remote) throw_al_exception("put: destination buffer is null (the peer attached no buffer)");
  comm.check_status();
  if (dest == comm.rank() && !comm.is_emulated()) {
    AL_CHECK_CUDA(cudaMemcpyAsync(dest_remote, src, bytes, cudaMemcpyDeviceToDevice, comm.get_stream()));
    return;
  }
  const int ctas = (int)std::max<size_t>(1, std::min<size_t>((bytes + 65535) / 65536, (size_t)tuning().max_ctas));
  device::launch_put(dest_remote, src, bytes, ctas, comm.get_stream());
}

void get(void* dst, int src_rank, const void* src_remote, size_t bytes, DeviceCommunicator& comm) {
  if (src_rank < 0 || bytes == 0) return;
  if (!src_remote) throw_al_exception("get: source buffer is null (the peer attached no buffer)");
  comm.check_status();
  if (src_rank == comm.rank() && !comm.is_emulated()) {
    AL_CHECK_CUDA(cudaMemcpyAsync(dst, src_remote, bytes, cudaMemcpyDeviceToDevice, comm.get_stream()));
    return;
  }
  // The same copy kernel as put with the roles of the pointers exchanged: remote loads, local stores.
  // More CTAs than a put of the same size: a load over NVLink occupies its thread for the round trip.
  const int ctas = (int)std::max<size_t>(1, std::min<size_t>((bytes + 32767) / 32768, (size_t)tuning().max_ctas));
  device::launch_put(dst, src_remote, bytes, ctas, comm.get_stream());
}

}  // namespace rma
}  // namespace internal
}  // namespace Al
