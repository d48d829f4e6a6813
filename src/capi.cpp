// C interface (see al/al_c.h): thin wrappers that translate exceptions into
// error codes and raw arrays into the C++ argument structures.
#include "al/al_c.h"

#include <algorithm>
#include <sstream>

#include "Al.hpp"
#include "al/device/kernels.hpp"
#include "al/tuning.hpp"

using namespace Al;
using namespace Al::internal;

namespace {

thread_local std::string g_err;

template <typename F>
int guard(F&& f) {
  try {
    f();
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return 1;
  } catch (...) {
    g_err = "unknown error";
    return 1;
  }
}

std::vector<size_t> vec(const size_t* p, size_t n) { return p ? std::vector<size_t>(p, p + n) : std::vector<size_t>(); }

Resolved resolve(int kind, DType dt, const void* send, void* recv, size_t count, int op, int root, int inplace,
                 int vector, const size_t* sc, const size_t* sd, const size_t* rc, const size_t* rd, int rank, int size) {
  const void* s = inplace ? in_place_ptr() : send;
  if ((OpKind)kind == OpKind::barrier) return Resolved();
  if (vector)
    return resolve_vector((OpKind)kind, dt, s, recv, vec(sc, (size_t)size), vec(sd, (size_t)size), vec(rc, (size_t)size),
                          vec(rd, (size_t)size), (ReductionOperator)op, root, rank, size);
  return resolve_uniform((OpKind)kind, dt, s, recv, count, (ReductionOperator)op, root, rank, size);
}

cudaStream_t pick_stream(DeviceCommunicator* c, void* stream) {
  return stream == AL_C_COMM_STREAM ? c->get_stream() : (cudaStream_t)stream;
}

}  // namespace

extern "C" {

const char* al_last_error(void) { return g_err.c_str(); }
int al_init(void) { return guard([] { Initialize(); }); }
int al_finalize(void) { return guard([] { Finalize(); }); }
int al_initialized(void) { return Initialized() ? 1 : 0; }
int al_world_rank(void) { int r = -1; guard([&] { r = get_world()->rank(); }); return r; }
int al_world_size(void) { int r = -1; guard([&] { r = get_world()->size(); }); return r; }
int al_world_local_rank(void) { int r = -1; guard([&] { r = get_world()->local_rank(); }); return r; }
int al_world_local_size(void) { int r = -1; guard([&] { r = get_world()->local_size(); }); return r; }
int al_world_peer_alive(int world_rank) {
  int r = -1;
  guard([&] {
    World* w = get_world();
    if (world_rank < 0 || world_rank >= w->size()) throw_al_exception("world rank ", world_rank, " out of range");
    r = w->peer_alive(world_rank) ? 1 : 0;
  });
  return r;
}
int al_world_num_nodes(void) { int r = -1; guard([&] { r = get_world()->num_nodes(); }); return r; }
int al_world_node_index(void) { int r = -1; guard([&] { r = get_world()->node_index(get_world()->rank()); }); return r; }
int al_cuda_available(void) { return cuda::device_usable() ? 1 : 0; }

int al_info(char* buf, size_t buflen) {
  return guard([&] {
    std::ostringstream ss;
    ss << "Aluminum-B200 " << AL_VERSION << "\nBackends: host device host-transfer rma\n"
       << "nvtx: " << (profiling::nvtx_available() ? "found" : "not found") << "\n--- tuning ---\n"
       << tuning().describe();
    if (Initialized()) {
      World* w = get_world();
      ss << "--- world ---\n"
         << "rank " << w->rank() << " of " << w->size() << ", local rank " << w->local_rank() << " of " << w->local_size()
         << ", node " << w->node_index(w->rank()) << " of " << w->num_nodes() << " (" << w->node_of(w->rank()) << ")\n";
    }
    ss << "--- topology ---\n";
    if (cuda::device_usable()) ss << device::discover_topology().describe();
    else ss << "no CUDA device usable in this process\n";
    const std::string s = ss.str();
    if (buflen) {
      const size_t n = std::min(buflen - 1, s.size());
      memcpy(buf, s.data(), n);
      buf[n] = 0;
    }
  });
}

#define AL_TUNE_FIELDS(X)                                                                                      \
  X(pe_num_concurrent_ops) X(pe_hang_seconds) X(host_stage_bytes) X(host_mailbox_bytes) X(host_wait_timeout_s) \
  X(dev_stage_bytes) X(dev_mailbox_bytes) X(dev_wait_timeout_ms) X(dev_enable_nvls)   \
  X(max_ctas) X(max_ctas_nvls) X(max_ctas_zero_copy) X(threads_per_cta) X(debug_checks) X(debug_guard) X(stream_pool_size)    \
  X(disable_background_streams) X(host_serialize) X(host_two_level) X(host_two_level_max_bytes) X(fault_rank) X(fault_op) X(fault_kind) X(fault_delay_ms) X(fault_jitter_us) \
  X(p2p_max_ctas) X(bulk_pipeline) X(bulk_pub_ctas) X(bulk_con_ctas) X(ll_max_ctas) X(dev_mailbox_slots) X(p2p_rendezvous_bytes) X(p2p_ll_max_bytes) X(nvls_chunk_bytes) X(max_ctas_pipelined) X(window_enable) X(window_ctas) X(window_multimem) X(window_multimem_ag_ranks) X(window_rs_min_ranks) X(window_rs_min_bytes)

namespace {
/** "ll_max_bytes" or "ll_max_bytes@4" -> member pointer and row (-1 = all rows); nullptr if not a crossover. */
size_t Crossovers::*crossover_field(const std::string& full, int* row) {
  std::string n = full;
  *row = -1;
  const size_t at = n.find('@');
  if (at != std::string::npos) {
    const int p = atoi(n.c_str() + at + 1);
    *row = p <= 2 ? 0 : (p <= 4 ? 1 : 2);
    n = n.substr(0, at);
  }
  if (n == "ll_max_bytes") return &Crossovers::ll_max_bytes;
  if (n == "ar_oneshot_max_bytes") return &Crossovers::ar_oneshot_max_bytes;
  if (n == "ar_nvls_min_bytes") return &Crossovers::ar_nvls_min_bytes;
  if (n == "ar_pipeline_min_bytes") return &Crossovers::ar_pipeline_min_bytes;
  if (n == "nvls_pipeline_min_bytes") return &Crossovers::nvls_pipeline_min_bytes;
  if (n == "pipeline_min_bytes") return &Crossovers::pipeline_min_bytes;
  if (n == "window_min_bytes") return &Crossovers::window_min_bytes;
  if (n == "rs_nvls_min_bytes") return &Crossovers::rs_nvls_min_bytes;
  if (n == "ar_ll2_max_bytes") return &Crossovers::ar_ll2_max_bytes;
  if (n == "ar_ll_max_bytes") return &Crossovers::ar_ll_max_bytes;
  return nullptr;
}
}  // namespace

int al_set_tuning(const char* name, double value) {
  return guard([&] {
    const std::string n = name;
    Tuning& t = tuning();
    int row = -1;
    if (auto f = crossover_field(n, &row)) {
      for (int r = 0; r < 3; ++r)
        if (row < 0 || row == r) t.cross[r].*f = (size_t)value;
      return;
    }
#define X(f) if (n == #f) { t.f = (decltype(t.f))value; return; }
    AL_TUNE_FIELDS(X)
#undef X
    throw_al_exception("unknown tuning entry ", n);
  });
}

double al_get_tuning(const char* name) {
  const std::string n = name;
  const Tuning& t = tuning();
  int row = -1;
  if (auto f = crossover_field(n, &row)) return (double)(t.cross[row < 0 ? 2 : row].*f);  // no row given: 5-8 ranks
#define X(f) if (n == #f) return (double)t.f;
  AL_TUNE_FIELDS(X)
#undef X
  return -1;
}

void al_trace_enable(int on) { trace::enable(on != 0); }
void al_trace_clear(void) { trace::clear(); }
int al_trace_snapshot(char* buf, size_t buflen) {
  return guard([&] {
    std::string s;
    for (auto& l : trace::snapshot()) { s += l; s += "\n"; }
    if (buflen) {
      const size_t n = std::min(buflen - 1, s.size());
      memcpy(buf, s.data(), n);
      buf[n] = 0;
    }
  });
}

// ---------------------------------------------------------------- host backend
void* al_host_comm_create(void) {
  void* r = nullptr;
  guard([&] { r = new HostCommunicator(); });
  return r;
}
void* al_host_comm_create_group(const int* world_ranks, int n) {
  void* r = nullptr;
  guard([&] {
    if (!world_ranks || n < 1) throw_al_exception("a group needs at least one world rank");
    r = new HostCommunicator(HostCommunicator::from_ranks(std::vector<int>(world_ranks, world_ranks + n)));
  });
  return r;
}
void* al_host_comm_split(void* comm, int color, int key) {
  void* r = nullptr;
  guard([&] { r = new HostCommunicator(((HostCommunicator*)comm)->split(color, key)); });
  return r;
}
void al_host_comm_destroy(void* comm) { delete (HostCommunicator*)comm; }
int al_host_comm_rank(void* comm) { return ((HostCommunicator*)comm)->rank(); }
int al_host_comm_size(void* comm) { return ((HostCommunicator*)comm)->size(); }
int al_host_comm_local_rank(void* comm) { return ((HostCommunicator*)comm)->local_rank(); }
int al_host_comm_local_size(void* comm) { return ((HostCommunicator*)comm)->local_size(); }
void* al_host_comm_local(void* comm) {
  void* r = nullptr;
  guard([&] { r = new HostCommunicator(((HostCommunicator*)comm)->local()); });
  return r;
}
int al_host_comm_stats(void* comm, uint64_t* out) {
  return guard([&] {
    host::CommStats s = ((HostCommunicator*)comm)->stats();
    out[0] = s.collectives; out[1] = s.p2p_ops; out[2] = s.bytes; out[3] = s.failures;
  });
}
int al_host_comm_abort(void* comm, const char* why) {
  return guard([&] { ((HostCommunicator*)comm)->abort(why ? why : "aborted by the caller"); });
}

int al_host_collective(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op, int root,
                       int inplace, int vector, const size_t* sc, const size_t* sd, const size_t* rc, const size_t* rd,
                       void** req_out) {
  return guard([&] {
    HostCommunicator& c = *(HostCommunicator*)comm;
    Resolved r = resolve(kind, (DType)dtype, send, recv, count, op, root, inplace, vector, sc, sd, rc, rd, c.rank(), c.size());
    if (trace::enabled()) trace::record_op("HostBackend", (DType)dtype, op_kind_name((OpKind)kind), c.rank(), c.size(), count);
    if (req_out) {
      auto* req = new HostBackend::req_type();
      try { HostBackend::run(std::move(r), c, req); } catch (...) { delete req; throw; }
      *req_out = req;
    } else {
      HostBackend::run(std::move(r), c, nullptr);
    }
  });
}

int al_host_p2p(void* comm, int n, const int* is_send, const int* peer, void* const* buf, const size_t* bytes,
                void** req_out) {
  return guard([&] {
    HostCommunicator& c = *(HostCommunicator*)comm;
    std::vector<host::P2PItem> items;
    for (int i = 0; i < n; ++i)
      items.push_back(is_send[i] ? HostBackend::make_send(buf[i], bytes[i], peer[i]) : HostBackend::make_recv(buf[i], bytes[i], peer[i]));
    if (req_out) {
      auto* req = new HostBackend::req_type();
      try { HostBackend::run_p2p(std::move(items), c, req, "p2p"); } catch (...) { delete req; throw; }
      *req_out = req;
    } else {
      HostBackend::run_p2p(std::move(items), c, nullptr, "p2p");
    }
  });
}

int al_host_test(void** req, int* done) {
  return guard([&] {
    *done = 1;
    if (!req || !*req) return;
    auto* r = (HostBackend::req_type*)*req;
    bool d;
    try { d = HostBackend::test(*r); } catch (...) { delete r; *req = nullptr; throw; }
    *done = d ? 1 : 0;
    if (d) { delete r; *req = nullptr; }
  });
}

int al_host_wait(void** req) {
  return guard([&] {
    if (!req || !*req) return;
    auto* r = (HostBackend::req_type*)*req;
    *req = nullptr;
    std::unique_ptr<HostBackend::req_type> hold(r);
    HostBackend::wait(*r);
  });
}

// -------------------------------------------------------------- device backend
void* al_dev_comm_create(void* stream) {
  void* r = nullptr;
  guard([&] { r = new DeviceCommunicator((cudaStream_t)stream); });
  return r;
}
void* al_dev_comm_create_group(const int* world_ranks, int n, void* stream) {
  void* r = nullptr;
  guard([&] {
    if (!world_ranks || n < 1) throw_al_exception("a group needs at least one world rank");
    r = new DeviceCommunicator(DeviceCommunicator::from_ranks(std::vector<int>(world_ranks, world_ranks + n), (cudaStream_t)stream));
  });
  return r;
}
void* al_dev_comm_create_emulated(int p, void* stream) {
  void* r = nullptr;
  guard([&] { r = new DeviceCommunicator(DeviceCommunicator::emulated(p, (cudaStream_t)stream)); });
  return r;
}
void* al_dev_comm_split(void* comm, int color, int key, void* stream) {
  void* r = nullptr;
  guard([&] { r = new DeviceCommunicator(((DeviceCommunicator*)comm)->split(color, key, (cudaStream_t)stream)); });
  return r;
}
void al_dev_comm_destroy(void* comm) { delete (DeviceCommunicator*)comm; }
int al_dev_comm_rank(void* comm) { return ((DeviceCommunicator*)comm)->rank(); }
int al_dev_comm_size(void* comm) { return ((DeviceCommunicator*)comm)->size(); }
int al_dev_comm_nlocal(void* comm) {
  auto* c = (DeviceCommunicator*)comm;
  return c->is_emulated() ? c->size() : 1;
}
int al_dev_comm_has_multicast(void* comm) { return ((DeviceCommunicator*)comm)->has_multicast() ? 1 : 0; }
const char* al_dev_comm_backing(void* comm) { return ((DeviceCommunicator*)comm)->memory_backing(); }
int al_dev_comm_set_timeout_ms(void* comm, double ms) {
  return guard([&] { ((DeviceCommunicator*)comm)->set_wait_timeout_ms(ms); });
}
int al_dev_comm_abort(void* comm, const char* why) {
  return guard([&] { ((DeviceCommunicator*)comm)->abort(why ? why : "aborted by the caller"); });
}
int al_dev_comm_stats(void* comm, uint64_t* out) {
  return guard([&] {
    device::CommStats s = ((DeviceCommunicator*)comm)->stats();
    out[0] = s.ops; out[1] = s.bytes; out[2] = s.kernels; out[3] = s.timeouts;
    out[4] = s.ar_one_shot; out[5] = s.ar_two_shot; out[6] = s.ar_nvls; out[7] = s.ar_nvls_zero_copy;
    out[8] = s.bulk_pipeline; out[9] = s.window; out[10] = s.ll; out[11] = s.rows; out[12] = s.rs_nvls;
  });
}
int al_dev_comm_status(void* comm, uint64_t* out) {
  device::DeviceStatus s = ((DeviceCommunicator*)comm)->status();
  out[0] = s.code; out[1] = s.rank; out[2] = s.peer; out[3] = s.where; out[4] = s.epoch; out[5] = s.seen;
  return 0;
}

int al_dev_collective(void* comm, int kind, int nlocal, const void* const* send, void* const* recv, size_t count,
                      int dt_in, int dt_wire, int dt_out, int op, int root, int inplace, int vector, const size_t* sc,
                      const size_t* sd, const size_t* rc, const size_t* rd, double scale, int algo, int ctas, void* stream,
                      void** req_out) {
  return guard([&] {
    DeviceCommunicator& c = *(DeviceCommunicator*)comm;
    ScopedDevice on_device(c.device());
    const int p = c.size();
    const int expect = c.is_emulated() ? p : 1;
    if (nlocal != expect) throw_al_exception("expected ", expect, " local rank(s), got ", nlocal);
    device::CollDesc d;
    d.kind = (device::DevColl)kind;
    d.in = (DType)dt_in;
    d.wire = dt_wire < 0 ? d.in : (DType)dt_wire;
    d.out = dt_out < 0 ? d.in : (DType)dt_out;
    d.op = (ReductionOperator)op;
    d.root = root;
    d.count = count;
    d.vector = vector != 0;
    d.scale = scale;
    if ((OpKind)kind == OpKind::allreduce) d.algo = (device::AllreduceAlgo)algo;
    else d.path = (device::CollPath)algo;
    d.ctas = ctas;
    std::vector<device::RankArgs> ra((size_t)nlocal);
    for (int lr = 0; lr < nlocal; ++lr) {
      const int rank = c.is_emulated() ? lr : c.rank();
      const size_t row = (size_t)lr * (size_t)p;
      // Pointer arithmetic of in-place forms uses the element size of the buffer it applies to.
      Resolved r = resolve(kind, (OpKind)kind == OpKind::allgather || (OpKind)kind == OpKind::gather ? d.out : d.in,
                           send ? send[lr] : nullptr, recv ? recv[lr] : nullptr, count, op, root, inplace, vector,
                           sc ? sc + row : nullptr, sd ? sd + row : nullptr, rc ? rc + row : nullptr,
                           rd ? rd + row : nullptr, rank, p);
      ra[(size_t)lr].send = r.send;
      ra[(size_t)lr].recv = r.recv;
      ra[(size_t)lr].send_counts = std::move(r.send_counts);
      ra[(size_t)lr].send_displs = std::move(r.send_displs);
      ra[(size_t)lr].recv_counts = std::move(r.recv_counts);
      ra[(size_t)lr].recv_displs = std::move(r.recv_displs);
    }
    if (trace::enabled()) trace::record_op("DeviceBackend", d.in, op_kind_name((OpKind)kind), c.rank(), p, count);
    if (req_out) {
      cudaStream_t s = device::begin_nonblocking(c);
      c.collective(d, ra, s);
      *req_out = new device::Request(device::end_nonblocking(c, s));
    } else {
      c.collective(d, ra, pick_stream(&c, stream));
    }
  });
}

int al_dev_latency_breakdown(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op,
                             int algo, int warmup, int iters, void* stream, double* out_us) {
  return guard([&] {
    DeviceCommunicator& c = *(DeviceCommunicator*)comm;
    if (c.is_emulated()) throw_al_exception("al_dev_latency_breakdown: not for emulated communicators");
    cudaStream_t s = pick_stream(&c, stream);
    cudaEvent_t e0, e1;
    AL_CHECK_CUDA(cudaEventCreate(&e0));
    AL_CHECK_CUDA(cudaEventCreate(&e1));
    c.enable_stamps(true);
    const void* sp[1] = {send};
    void* rp[1] = {recv};
    std::vector<double> col[6];
    // The ranks start every call together: a barrier on shared memory (the control plane's socket exchange
    // releases the ranks one after the other, and that skew would end up inside the timed interval).
    HostCommunicator start_line(c.group());
    for (int i = 0; i < warmup + iters; ++i) {
      Barrier<HostBackend>(start_line);
      AL_CHECK_CUDA(cudaEventRecord(e0, s));
      const double h0 = get_time();
      if (al_dev_collective(comm, kind, 1, sp, rp, count, dtype, -1, -1, op, 0, 0, 0, nullptr, nullptr, nullptr, nullptr,
                            1.0, algo, 0, (void*)s, nullptr) != 0)
        throw_al_exception(g_err);
      const double h1 = get_time();
      AL_CHECK_CUDA(cudaEventRecord(e1, s));
      AL_CHECK_CUDA(cudaEventSynchronize(e1));
      float ms = 0;
      AL_CHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
      uint64_t t[4];
      c.read_stamps(t);
      if (i < warmup) continue;
      col[0].push_back(ms * 1e3);
      col[1].push_back((h1 - h0) * 1e6);
      col[2].push_back((double)(t[1] - t[0]) * 1e-3);
      col[3].push_back((double)(t[2] - t[1]) * 1e-3);
      col[4].push_back((double)(t[3] - t[2]) * 1e-3);
      col[5].push_back((double)(t[3] - t[0]) * 1e-3);
    }
    c.enable_stamps(false);
    for (int k = 0; k < 6; ++k) {
      std::sort(col[k].begin(), col[k].end());
      out_us[k] = col[k].empty() ? 0.0 : col[k][col[k].size() / 2];
    }
    AL_CHECK_CUDA(cudaEventDestroy(e0));
    AL_CHECK_CUDA(cudaEventDestroy(e1));
  });
}

int al_dev_exchange_rows(void* comm, int nlocal, const void* const* send, void* const* recv, const long long* const* send_idx,
                         const long long* const* recv_idx, size_t row_bytes, size_t send_row_stride, size_t recv_row_stride,
                         const size_t* send_rows, const size_t* send_first, const size_t* send_peer_off,
                         const size_t* recv_rows, const size_t* recv_first, const size_t* recv_peer_off, void* stream,
                         void** req_out) {
  return guard([&] {
    DeviceCommunicator& c = *(DeviceCommunicator*)comm;
    ScopedDevice on_device(c.device());
    const size_t p = (size_t)c.size();
    std::vector<device::RowArgs> ra((size_t)nlocal);
    for (int lr = 0; lr < nlocal; ++lr) {
      device::RowArgs& a = ra[(size_t)lr];
      a.send = send[lr];
      a.recv = recv[lr];
      a.send_idx = send_idx ? send_idx[lr] : nullptr;
      a.recv_idx = recv_idx ? recv_idx[lr] : nullptr;
      const size_t row = (size_t)lr * p;
      a.send_rows.assign(send_rows + row, send_rows + row + p);
      a.send_first.assign(send_first + row, send_first + row + p);
      a.send_peer_off.assign(send_peer_off + row, send_peer_off + row + p);
      a.recv_rows.assign(recv_rows + row, recv_rows + row + p);
      a.recv_first.assign(recv_first + row, recv_first + row + p);
      a.recv_peer_off.assign(recv_peer_off + row, recv_peer_off + row + p);
    }
    if (trace::enabled()) trace::record_op("DeviceBackend", DType::u8, "exchange_rows", c.rank(), c.size(), row_bytes);
    if (req_out) {
      cudaStream_t s = device::begin_nonblocking(c);
      c.exchange_rows(ra, row_bytes, send_row_stride, recv_row_stride, s);
      *req_out = new device::Request(device::end_nonblocking(c, s));
    } else {
      c.exchange_rows(ra, row_bytes, send_row_stride, recv_row_stride, pick_stream(&c, stream));
    }
  });
}

int al_dev_register(void* comm, void* ptr, size_t bytes) {
  int w = -1;
  if (guard([&] { w = ((DeviceCommunicator*)comm)->register_buffer(ptr, bytes); }) != 0) return -2;
  return w;
}
int al_dev_register_emulated(void* comm, void* const* ptrs, int n, size_t bytes) {
  int w = -1;
  if (guard([&] { w = ((DeviceCommunicator*)comm)->register_buffers_emulated(std::vector<void*>(ptrs, ptrs + n), bytes); }) != 0)
    return -2;
  return w;
}
int al_dev_unregister(void* comm, void* ptr) {
  return guard([&] { ((DeviceCommunicator*)comm)->unregister_buffer(ptr); });
}

int al_dev_time_collective(void* comm, int kind, const void* send, void* recv, size_t count, int dtype, int op,
                           int warmup, int iters, void* stream, float* out_ms) {
  return guard([&] {
    DeviceCommunicator& c = *(DeviceCommunicator*)comm;
    if (c.is_emulated()) throw_al_exception("al_dev_time_collective: not for emulated communicators");
    cudaStream_t s = pick_stream(&c, stream);
    cudaEvent_t e0, e1;
    AL_CHECK_CUDA(cudaEventCreate(&e0));
    AL_CHECK_CUDA(cudaEventCreate(&e1));
    const void* sp[1] = {send};
    void* rp[1] = {recv};
    // host barrier on shared memory before every call, as in benchmark_ops (see al_dev_latency_breakdown)
    HostCommunicator start_line(c.group());
    for (int i = 0; i < warmup + iters; ++i) {
      Barrier<HostBackend>(start_line);
      AL_CHECK_CUDA(cudaEventRecord(e0, s));
      if (al_dev_collective(comm, kind, 1, sp, rp, count, dtype, -1, -1, op, 0, 0, 0, nullptr, nullptr, nullptr, nullptr,
                            1.0, 0, 0, (void*)s, nullptr) != 0)
        throw_al_exception(g_err);
      AL_CHECK_CUDA(cudaEventRecord(e1, s));
      AL_CHECK_CUDA(cudaEventSynchronize(e1));
      float ms = 0;
      AL_CHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
      if (i >= warmup) out_ms[i - warmup] = ms;
    }
    AL_CHECK_CUDA(cudaEventDestroy(e0));
    AL_CHECK_CUDA(cudaEventDestroy(e1));
  });
}

int al_dev_p2p(void* comm, int n, const int* is_send, const int* peer, const int* owner, void* const* buf,
               const size_t* bytes, void* stream, void** req_out) {
  return guard([&] {
    DeviceCommunicator& c = *(DeviceCommunicator*)comm;
    ScopedDevice on_device(c.device());
    std::vector<device::P2PDesc> items((size_t)n);
    for (int i = 0; i < n; ++i) {
      items[(size_t)i].is_send = is_send[i] != 0;
      items[(size_t)i].peer = peer[i];
      items[(size_t)i].owner = owner ? owner[i] : -1;
      items[(size_t)i].bytes = bytes[i];
      if (is_send[i]) items[(size_t)i].sbuf = buf[i];
      else items[(size_t)i].rbuf = buf[i];
    }
    if (req_out) {
      cudaStream_t s = device::begin_nonblocking(c);
      c.p2p(items, s);
      *req_out = new device::Request(device::end_nonblocking(c, s));
    } else {
      c.p2p(items, pick_stream(&c, stream));
    }
  });
}

int al_dev_test(void** req, int* done) {
  return guard([&] {
    *done = 1;
    if (!req || !*req) return;
    auto* r = (device::Request*)*req;
    const bool d = device::test_request(*r);
    *done = d ? 1 : 0;
    if (d) { delete r; *req = nullptr; }
  });
}

int al_dev_wait(void** req) {
  return guard([&] {
    if (!req || !*req) return;
    std::unique_ptr<device::Request> r((device::Request*)*req);
    *req = nullptr;
    device::wait_request(*r);
  });
}

void* al_dev_symm_alloc(void* comm, size_t bytes) {
  void* r = nullptr;
  guard([&] { r = ((DeviceCommunicator*)comm)->symm_alloc(bytes); });
  return r;
}
int al_dev_check_guards(void* comm) { return guard([&] { ((DeviceCommunicator*)comm)->check_guards(); }); }
int al_dev_symm_free(void* comm, void* ptr) { return guard([&] { ((DeviceCommunicator*)comm)->symm_free(ptr); }); }
void* al_dev_symm_peer_ptr(void* comm, void* local_ptr, int peer) {
  void* r = nullptr;
  guard([&] {
    auto* c = (DeviceCommunicator*)comm;
    size_t off = 0;
    if (!c->find_symm(local_ptr, 1, &off)) throw_al_exception("pointer is not inside a symmetric allocation");
    r = c->symm_peer_ptr(c->symm_index(local_ptr), peer, off);
  });
  return r;
}

// ------------------------------------------------------------------ RMA / halo
void* al_rma_attach(void* comm, void* local_buf, int peer) {
  void* r = nullptr;
  guard([&] { r = rma::attach(local_buf, peer, *(DeviceCommunicator*)comm); });
  return r;
}
int al_rma_detach(void* comm, void* remote_buf, int peer) {
  return guard([&] { rma::detach(remote_buf, peer, *(DeviceCommunicator*)comm); });
}
int al_rma_put(void* comm, const void* src, int dest, void* dest_remote, size_t bytes) {
  return guard([&] { rma::put(src, dest, dest_remote, bytes, *(DeviceCommunicator*)comm); });
}
int al_rma_get(void* comm, void* dst, int src_rank, const void* src_remote, size_t bytes) {
  return guard([&] { rma::get(dst, src_rank, src_remote, bytes, *(DeviceCommunicator*)comm); });
}
int al_rma_notify(void* comm, int peer) { return guard([&] { rma::notify(peer, *(DeviceCommunicator*)comm); }); }
int al_rma_wait(void* comm, int peer) { return guard([&] { rma::wait(peer, *(DeviceCommunicator*)comm); }); }
int al_rma_sync(void* comm, int peer) { return guard([&] { ext::Sync(peer, *(DeviceCommunicator*)comm); }); }

int al_halo_exchange(void* comm, float* const* tensors, size_t nc, size_t d_local, size_t plane, size_t depth,
                     int periodic, int ctas, void* stream) {
  return guard([&] {
    DeviceCommunicator& c = *(DeviceCommunicator*)comm;
    c.check_status();
    const int p = c.size();
    device::HaloParams P{};
    P.ws = c.workspace();
    for (int r = 0; r < p; ++r) {
      P.tensor[r] = tensors[r];
      P.lo[r] = r > 0 ? r - 1 : (periodic && p > 1 ? p - 1 : -1);
      P.hi[r] = r + 1 < p ? r + 1 : (periodic && p > 1 ? 0 : -1);
    }
    P.nc = nc; P.d_local = d_local; P.plane = plane; P.depth = depth;
    P.epoch = c.next_halo_epoch();
    P.timeout_ns = c.wait_timeout_ns();
    const int nlocal = c.is_emulated() ? p : 1;
    P.rank0 = c.is_emulated() ? 0 : c.rank();
    if (ctas <= 0) ctas = tuning().max_ctas;
    if (nlocal > 1) ctas = std::max(1, std::min(ctas, 148 / nlocal));
    device::launch_halo_exchange(P, ctas, 512, nlocal, pick_stream(&c, stream));
  });
}

int al_halo_pack(float* packed, const float* tensor, size_t nc, size_t d_total, size_t plane, size_t d_first,
                 size_t depth, int unpack, void* stream) {
  return guard([&] {
    if (unpack) device::launch_halo_unpack(const_cast<float*>(tensor), packed, nc, d_total, plane, d_first, depth, (cudaStream_t)stream);
    else device::launch_halo_pack(packed, tensor, nc, d_total, plane, d_first, depth, (cudaStream_t)stream);
  });
}

// --------------------------------------------------------------- element-wise
int al_scale_cast(void* out, int out_dt, const void* in, int in_dt, size_t n, double scale, void* stream) {
  return guard([&] { device::launch_scale_cast(out, (DType)out_dt, in, (DType)in_dt, n, scale, (cudaStream_t)stream); });
}
int al_sgd_momentum(float* param, float* momentum, float* grad, size_t n, float lr, float mu, float weight_decay,
                    float grad_scale, int first_step, int zero_grad, void* stream) {
  return guard([&] {
    device::launch_sgd_momentum(param, momentum, grad, n, lr, mu, weight_decay, grad_scale, first_step, zero_grad, (cudaStream_t)stream);
  });
}
int al_fill_u32(void* out, size_t n, uint32_t value, void* stream) {
  return guard([&] { device::launch_fill_u32((uint32_t*)out, n, value, (cudaStream_t)stream); });
}

}  // extern "C"
