// Device communicator: workspace set-up, algorithm / grid selection, launch
// ordering and failure reporting (see al/device/communicator.hpp).
#include "al/device/communicator.hpp"

#include <algorithm>
#include <atomic>
#include <mutex>

#include "al/device/kernels.hpp"
#include "al/rma.hpp"
#include "al/runtime.hpp"
#include "al/trace.hpp"
#include "al/tuning.hpp"
#include "al/util/meta.hpp"

namespace Al {

using namespace internal;
using namespace internal::device;

struct DeviceCommunicator::Impl {
  int p = 1, rank0 = 0, nlocal = 1;
  bool emulated = false;
  int device = 0, sm_count = 148;
  std::unique_ptr<SymmBlock> block;
  Workspace ws{};
  DeviceStatus* status_host = nullptr;
  uint64_t seq = 0;
  uint64_t halo_epoch = 0;
  uint64_t timeout_ns = 0;
  cudaStream_t last_stream = nullptr;
  bool have_last = false;
  cudaEvent_t chain_event = nullptr;
  std::vector<uint64_t> p2p_sent, p2p_recvd;  // [nlocal][p]
  std::vector<std::unique_ptr<SymmBlock>> user_blocks;
  std::vector<size_t> user_guard;  // bytes of guard region before and after the user's part of each block (0: none)
  size_t guard_of(const SymmBlock* b) const {
    for (size_t i = 0; i < user_blocks.size(); ++i)
      if (user_blocks[i].get() == b) return user_guard[i];
    return 0;
  }
  // Registered buffers.  Slot w describes window w on every rank; the device copy is what kernels read.
  struct Window {
    bool used = false;
    void* local[kMaxRanks] = {};       // start of each LOCAL rank's buffer (index = rank; one entry outside emulation)
    const SymmBlock* block = nullptr;  // set when the window is a whole symm_alloc block
    std::vector<void*> opened;         // CUDA IPC mappings to close
  };
  Window windows[kMaxWindows];
  WindowTable table_host{};
  WindowTable* table_dev = nullptr;
  CommStats stats;
  std::atomic<bool> aborted{false};
  std::string abort_msg;
  std::mutex mu;

  size_t off_stage() const { return FlagLayout::bytes; }
  size_t off_mbox() const { return FlagLayout::bytes + 2 * ws.half_bytes; }
  size_t off_ll() const { return off_mbox() + (size_t)p * (size_t)ws.mbox_slots * ws.mbox_slot_bytes; }
  uint64_t p2p_launches = 0;
  uint64_t* stamps_dev = nullptr;

  void setup(std::unique_ptr<SymmBlock> b, int p_, int rank0_, int nlocal_) {
    p = p_; rank0 = rank0_; nlocal = nlocal_;
    block = std::move(b);
    AL_CHECK_CUDA(cudaGetDevice(&device));
    AL_CHECK_CUDA(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device));
    ws.p = p;
    for (int r = 0; r < p; ++r) {
      char* base = (char*)block->peer(r);
      ws.flags[r] = (uint64_t*)base;
      ws.stage[r] = base + off_stage();
      ws.mbox[r] = base + off_mbox();
      ws.ll[r] = base + off_ll();
    }
    ws.mc_stage = block->mc() ? (char*)block->mc() + off_stage() : nullptr;
    void* hp = nullptr;
    AL_CHECK_CUDA(cudaHostAlloc(&hp, sizeof(DeviceStatus), cudaHostAllocMapped | cudaHostAllocPortable));
    memset(hp, 0, sizeof(DeviceStatus));
    status_host = (DeviceStatus*)hp;
    void* dp = nullptr;
    AL_CHECK_CUDA(cudaHostGetDevicePointer(&dp, hp, 0));
    ws.status = (DeviceStatus*)dp;
    timeout_ns = (uint64_t)(tuning().dev_wait_timeout_ms * 1e6);
    AL_CHECK_CUDA(cudaEventCreateWithFlags(&chain_event, cudaEventDisableTiming));
    AL_CHECK_CUDA(cudaMalloc((void**)&table_dev, sizeof(WindowTable)));
    AL_CHECK_CUDA(cudaMemset(table_dev, 0, sizeof(WindowTable)));
    p2p_sent.assign((size_t)nlocal * (size_t)p, 0);
    p2p_recvd.assign((size_t)nlocal * (size_t)p, 0);
  }

  ~Impl() {
    internal::rma::forget(this);
    for (auto& w : windows)
      for (void* m : w.opened) AL_WARN_CUDA(cudaIpcCloseMemHandle(m));
    if (table_dev) AL_WARN_CUDA(cudaFree(table_dev));
    if (stamps_dev) AL_WARN_CUDA(cudaFree(stamps_dev));
    if (chain_event) AL_WARN_CUDA(cudaEventDestroy(chain_event));
    if (status_host) AL_WARN_CUDA(cudaFreeHost(status_host));
  }

  static size_t block_bytes(int p, size_t half, size_t slot, int slots, size_t ll_slot) {
    return FlagLayout::bytes + 2 * half + (size_t)p * (size_t)slots * slot + kLLAreaBytes +
           (size_t)p * (size_t)slots * ll_slot;
  }

  int free_window() const {
    for (int w = 0; w < kMaxWindows; ++w)
      if (!windows[w].used) return w;
    return -1;
  }
  void push_table() {
    AL_CHECK_CUDA(cudaMemcpy(table_dev, &table_host, sizeof(WindowTable), cudaMemcpyHostToDevice));
  }
  void clear_window(int w) {
    for (void* m : windows[w].opened) AL_WARN_CUDA(cudaIpcCloseMemHandle(m));
    windows[w] = Window();
    for (int r = 0; r < kMaxRanks; ++r) { table_host.peer[w][r] = nullptr; table_host.bytes[w][r] = 0; }
    table_host.mc[w] = nullptr;
  }
  /** A whole symmetric block becomes window `w` (same slot on every rank: blocks are allocated collectively). */
  void add_block_window(const SymmBlock* b) {
    const int w = free_window();
    if (w < 0) return;
    Window& W = windows[w];
    W.used = true;
    W.block = b;
    for (int r = 0; r < p; ++r) {
      table_host.peer[w][r] = (char*)b->peer(r);
      table_host.bytes[w][r] = b->bytes();
    }
    for (int lr = 0; lr < nlocal; ++lr) W.local[rank0 + lr] = b->peer(rank0 + lr);
    table_host.mc[w] = (char*)b->mc();
    push_table();
  }

  /** Make `stream` wait for the communicator's previous operation if that ran on another stream. */
  void order_after_previous(cudaStream_t stream) {
    if (have_last && last_stream != stream) {
      AL_CHECK_CUDA(cudaEventRecord(chain_event, last_stream));
      AL_CHECK_CUDA(cudaStreamWaitEvent(stream, chain_event, 0));
    }
    last_stream = stream;
    have_last = true;
  }
};

namespace {

size_t half_bytes_cfg() { return tuning().dev_stage_bytes / 4096 * 4096; }
size_t slot_bytes_cfg() { return std::max<size_t>(4096, tuning().dev_mailbox_bytes / 4096 * 4096); }
int slots_cfg() { return std::max(2, std::min(16, tuning().dev_mailbox_slots)); }
/** Packet slot of the point-to-point path: twice the largest payload (every 8 bytes carry 4 of payload). */
size_t p2p_ll_slot_cfg() { return 2 * round_up(std::min(tuning().p2p_ll_max_bytes, kP2PLLMaxPayloadBytes), (size_t)4096); }

void require_device() {
  if (!cuda::device_usable()) throw_al_exception("the device backend needs a CUDA device, none is usable in this process");
}

}  // namespace

DeviceCommunicator::DeviceCommunicator() : DeviceCommunicator((cudaStream_t) nullptr) {}

DeviceCommunicator::DeviceCommunicator(cudaStream_t stream)
    : DeviceCommunicator(Group::world_group(get_world()), stream) {}

DeviceCommunicator::DeviceCommunicator(const Group& group, cudaStream_t stream)
    : group_(group), stream_(stream), impl_(std::make_shared<Impl>()) {
  require_device();
  if (!group.single_node()) {
    // Peers' memory is mapped through descriptors passed between processes and reached over NVLink;
    // neither crosses a node boundary.
    for (int r = 0; r < group.size(); ++r)
      if (!group.world()->same_node(group.world_rank_of(r)))
        throw_al_exception("a device communicator spans one NVLink domain, but rank ", r, " is on node '",
                           group.world()->node_of(group.world_rank_of(r)),
                           "': split the communicator by node, or use the host-transfer backend across nodes");
  }
  const size_t half = half_bytes_cfg(), slot = slot_bytes_cfg();
  const int slots = slots_cfg();
  const size_t ll_slot = p2p_ll_slot_cfg();
  auto block = SymmBlock::create(group, Impl::block_bytes(group.size(), half, slot, slots, ll_slot), true);
  impl_->ws.half_bytes = half;
  impl_->ws.mbox_slot_bytes = slot;
  impl_->ws.mbox_slots = slots;
  impl_->ws.p2p_ll_slot_bytes = ll_slot;
  impl_->setup(std::move(block), group.size(), group.rank(), 1);
}

DeviceCommunicator::DeviceCommunicator(std::shared_ptr<Impl> impl, const Group& g, cudaStream_t s)
    : group_(g), stream_(s), impl_(std::move(impl)) {}

DeviceCommunicator DeviceCommunicator::emulated(int p, cudaStream_t stream) {
  require_device();
  auto impl = std::make_shared<Impl>();
  const size_t half = half_bytes_cfg(), slot = slot_bytes_cfg();
  const int slots = slots_cfg();
  const size_t ll_slot = p2p_ll_slot_cfg();
  auto block = SymmBlock::create_emulated(p, Impl::block_bytes(p, half, slot, slots, ll_slot));
  impl->ws.half_bytes = half;
  impl->ws.mbox_slot_bytes = slot;
  impl->ws.mbox_slots = slots;
  impl->ws.p2p_ll_slot_bytes = ll_slot;
  impl->emulated = true;
  impl->setup(std::move(block), p, 0, p);
  return DeviceCommunicator(std::move(impl), Group(), stream);
}

DeviceCommunicator DeviceCommunicator::from_ranks(const std::vector<int>& world_ranks, cudaStream_t stream) {
  return DeviceCommunicator(Group(get_world(), world_ranks), stream);
}

DeviceCommunicator::~DeviceCommunicator() = default;
DeviceCommunicator::DeviceCommunicator(DeviceCommunicator&&) noexcept = default;
DeviceCommunicator& DeviceCommunicator::operator=(DeviceCommunicator&&) noexcept = default;

DeviceCommunicator DeviceCommunicator::copy(cudaStream_t stream) const {
  if (impl_->emulated) return emulated(impl_->p, stream);
  return DeviceCommunicator(group_, stream);
}

DeviceCommunicator DeviceCommunicator::split(int color, int key, cudaStream_t stream) const {
  if (impl_->emulated) throw_al_exception("split is not available on an emulated communicator");
  return DeviceCommunicator(group_.split(color, key), stream);
}

int DeviceCommunicator::rank() const { return impl_->emulated ? 0 : impl_->rank0; }
int DeviceCommunicator::size() const { return impl_->p; }
bool DeviceCommunicator::is_emulated() const { return impl_->emulated; }
int DeviceCommunicator::device() const { return impl_->device; }
bool DeviceCommunicator::has_multicast() const { return impl_->ws.mc_stage != nullptr; }
const char* DeviceCommunicator::memory_backing() const { return impl_->block->backing(); }
const Workspace& DeviceCommunicator::workspace() const { return impl_->ws; }
uint64_t DeviceCommunicator::next_halo_epoch() { return ++impl_->halo_epoch; }

void DeviceCommunicator::enable_stamps(bool on) {
  Impl& I = *impl_;
  std::lock_guard<std::mutex> lock(I.mu);
  if (on && !I.stamps_dev) {
    AL_CHECK_CUDA(cudaMalloc((void**)&I.stamps_dev, 4 * sizeof(uint64_t)));
    AL_CHECK_CUDA(cudaMemset(I.stamps_dev, 0, 4 * sizeof(uint64_t)));
  }
  I.ws.stamps = on ? I.stamps_dev : nullptr;
}

void DeviceCommunicator::read_stamps(uint64_t out[4]) const {
  const Impl& I = *impl_;
  for (int i = 0; i < 4; ++i) out[i] = 0;
  if (!I.stamps_dev) return;
  AL_CHECK_CUDA(cudaDeviceSynchronize());
  AL_CHECK_CUDA(cudaMemcpy(out, I.stamps_dev, 4 * sizeof(uint64_t), cudaMemcpyDeviceToHost));
}

void DeviceCommunicator::set_wait_timeout_ms(double ms) {
  impl_->timeout_ns = (uint64_t)(std::max(0.001, ms) * 1e6);
}

DeviceStatus DeviceCommunicator::status() const {
  DeviceStatus s;
  memcpy(&s, (const void*)impl_->status_host, sizeof(s));
  s.code = __atomic_load_n(&impl_->status_host->code, __ATOMIC_ACQUIRE);
  return s;
}

void DeviceCommunicator::abort(const std::string& why) {
  std::lock_guard<std::mutex> lock(impl_->mu);
  if (!impl_->aborted.load()) { impl_->abort_msg = why; impl_->aborted.store(true); }
}

void DeviceCommunicator::check_status() const {
  if (impl_->aborted.load(std::memory_order_acquire))
    throw_al_exception("device communicator aborted: ", impl_->abort_msg, "; create a new one");
  const uint32_t code = __atomic_load_n(&impl_->status_host->code, __ATOMIC_ACQUIRE);
  if (code == kStatusOk) return;
  DeviceStatus s = status();
  static const char* where[] = {"data-ready flags", "reduced-slice flags", "closing barrier", "send credit",
                                "incoming data", "RMA / halo signal", "bulk copy completion", "protocol comparison"};
  if (code == kStatusMismatch) {
    static const char* proto[] = {"none", "staging", "NVLS through staging", "NVLS on symmetric buffers", "registered buffers (window)"};
    const unsigned mine = (unsigned)((s.epoch >> 8) & 0xff), theirs = (unsigned)((s.seen >> 8) & 0xff);
    throw_al_exception("device communicator failed: ranks ", s.rank, " and ", s.peer, " entered one operation on different "
                       "paths (", proto[mine < 5 ? mine : 0], " vs ", proto[theirs < 5 ? theirs : 0],
                       "): every rank must pass a registered / symmetric buffer, or none; the communicator is unusable, "
                       "create a new one");
  }
  impl_->stats.timeouts++;
  throw_al_exception("device communicator failed: rank ", s.rank, " timed out waiting for rank ", s.peer, " (",
                     where[s.where < 8 ? s.where : 0], ", epoch ", s.epoch, ", last seen ", s.seen,
                     "); the communicator is unusable, create a new one");
}

CommStats DeviceCommunicator::stats() const { return impl_->stats; }

// ---------------------------------------------------------------------------
// collectives
// ---------------------------------------------------------------------------
void DeviceCommunicator::collective(const CollDesc& d, const std::vector<RankArgs>& ranks, cudaStream_t stream) {
  Impl& I = *impl_;
  std::lock_guard<std::mutex> lock(I.mu);
  check_status();
  if ((int)ranks.size() != I.nlocal)
    throw_al_exception("expected arguments for ", I.nlocal, " local rank(s), got ", ranks.size());
  const int p = I.p;
  if (d.root < 0 || d.root >= p) throw_al_exception("root ", d.root, " out of range");

  const bool reduces = d.kind == DevColl::allreduce || d.kind == DevColl::reduce || d.kind == DevColl::reduce_scatter;
  DType in = d.in, wire = d.wire, out = d.out;
  size_t unit = 1;  // multiplier turning element counts into kernel counts
  if (!reduces && in == wire && wire == out) {
    unit = dtype_size(in);
    in = wire = out = DType::u8;  // pure data movement: count bytes
  }
  if (reduces && !collective_supported(in, wire, out, d.op))
    throw_al_exception("device backend: ", reduction_name(d.op), " on (", dtype_name(in), ", ", dtype_name(wire), ", ",
                       dtype_name(out), ") is not supported");
  if (!reduces && !(in == wire && wire == out) && !collective_supported(in, wire, out, ReductionOperator::sum))
    throw_al_exception("device backend: no kernel for this datatype conversion");

  // Small uniform allreduce / reduce_scatter / allgather / alltoall travel as low-latency packets.  This
  // is decided first, before anything else is prepared: these calls are all about the time the host spends
  // here.  Eligibility depends on facts every rank shares (operation, count, type), so the ranks agree.
  {
    const bool ll_kind = d.kind == DevColl::allreduce || d.kind == DevColl::reduce_scatter ||
                         d.kind == DevColl::allgather || d.kind == DevColl::alltoall;
    const size_t esz_ll = dtype_size(wire);
    const size_t pair_bytes = d.count * unit * esz_ll;  // what one rank sends to another
    const bool eligible = ll_kind && !d.vector && p > 1 && in == wire && wire == out && d.count > 0 &&
                          ll_supported(d.kind, wire, d.op);
    const bool fits = eligible && pair_bytes <= kLLPayloadBytes;
    // Allreduce beyond that: reduce-scatter and allgather in packets inside one kernel (two NVLink trips, 2(p-1)/p
    // of the vector per rank instead of p-1 times the vector); a slice must fit half a slot.
    const size_t slice_groups = ceil_div(ceil_div(pair_bytes, (size_t)16), (size_t)p);
    const bool fits2 = eligible && d.kind == DevColl::allreduce && p > 2 && slice_groups * 32 <= kLLSlotBytes / 2;
    const bool forced = d.kind == DevColl::allreduce ? d.algo == AllreduceAlgo::ll : d.path == CollPath::ll;
    const bool automatic = d.kind == DevColl::allreduce ? d.algo == AllreduceAlgo::automatic : d.path == CollPath::automatic;
    if (forced && !fits && !fits2)
      throw_al_exception("the low-latency path was requested but the operation does not qualify (uniform allreduce / "
                         "reduce_scatter / allgather / alltoall of at most ", kLLPayloadBytes, " bytes per pair of ranks)");
    const Tuning& tn = tuning();
    // One-phase packets cost an allreduce p-1 times the vector per rank: its limit is lower than that of the
    // other three operations (whose pair_bytes is one slice) and shrinks with the number of ranks.
    const size_t one_phase_max = d.kind == DevColl::allreduce
                                     ? std::min(tn.crossovers(p).ll_max_bytes, tn.crossovers(p).ar_ll_max_bytes)
                                     : tn.crossovers(p).ll_max_bytes;
    const bool one_phase = fits && ((forced && !(fits2 && pair_bytes > one_phase_max)) || (automatic && pair_bytes <= one_phase_max));
    const bool two_phase = !one_phase && fits2 && (forced || (automatic && pair_bytes <= tn.crossovers(p).ar_ll2_max_bytes));
    if (one_phase || two_phase) {
      LLParams L;
      L.two_phase = two_phase ? 1 : 0;
      L.ws = I.ws;
      for (int lr = 0; lr < I.nlocal; ++lr) {
        L.send[I.rank0 + lr] = ranks[(size_t)lr].send;
        L.recv[I.rank0 + lr] = ranks[(size_t)lr].recv;
      }
      L.count = d.count * unit;
      L.seq = ++I.seq;
      L.timeout_ns = I.timeout_ns;
      L.scale = d.scale;
      L.int_div = 1;
      if (d.op == ReductionOperator::avg) {
        if (dtype_is_float(wire)) L.scale *= 1.0 / p;
        else L.int_div = p;
      }
      L.kind = (int)d.kind;
      L.op = (int)d.op;
      L.rank0 = I.rank0;
      const size_t groups = ceil_div(pair_bytes, (size_t)16);
      int lctas = (int)std::max<size_t>(1, std::min<size_t>(ceil_div(groups, (size_t)256), (size_t)tn.ll_max_ctas));
      if (I.nlocal > 1) lctas = std::max(1, std::min(lctas, I.sm_count / I.nlocal));
      const int lthreads = groups <= 64 ? 64 : (groups <= 128 ? 128 : 256);
      I.order_after_previous(stream);
      I.stats.ops++;
      I.stats.bytes += pair_bytes;
      I.stats.kernels++;
      I.stats.ll++;
      launch_ll(L, wire, lctas, lthreads, I.nlocal, stream);
      return;
    }
  }

  CollParams P{};
  P.ws = I.ws;
  P.seq = ++I.seq;
  P.timeout_ns = I.timeout_ns;
  P.kind = (int)d.kind;
  P.op = (int)d.op;
  P.root = d.root;
  P.rank0 = I.rank0;
  P.count = d.count * unit;
  P.scale = d.scale;
  P.int_div = 1;
  if (d.op == ReductionOperator::avg) {
    if (dtype_is_float(wire)) P.scale *= 1.0 / p;
    else P.int_div = p;
  }

  const size_t esz = dtype_size(wire);
  const size_t half = I.ws.half_bytes;
  const size_t full_e = half / esz;
  const size_t cap_e = ((half / (size_t)p) / 256 * 256) / esz;           // one slot per source rank
  const size_t cap2_e = ((half / 2 / (size_t)p) / 256 * 256) / esz;      // two-phase allreduce
  size_t max_work_bytes = 0;

  // ---- algorithm -----------------------------------------------------------------
  const Tuning& tn = tuning();
  const Crossovers& X = tn.crossovers(p);
  const size_t bytes = P.count * esz;
  AllreduceAlgo algo = d.algo;
  bool zero_copy = false;
  const SymmBlock* sb_in = nullptr;
  const SymmBlock* sb_out = nullptr;
  size_t off_in = 0, off_out = 0;
  if (d.kind == DevColl::allreduce) {
    const bool nvls_ok = !I.emulated && p > 1 && I.ws.mc_stage != nullptr && in == wire && wire == out &&
                         nvls_allreduce_supported(wire, d.op);
    if (algo == AllreduceAlgo::nvls && !nvls_ok)
      throw_al_exception("NVLS allreduce requested but unavailable (no multicast, or type/operator unsupported)");
    if (nvls_ok && (algo == AllreduceAlgo::automatic || algo == AllreduceAlgo::nvls)) {
      const RankArgs& a = ranks[0];
      sb_in = find_symm(a.send, bytes, &off_in);
      sb_out = find_symm(a.recv, bytes, &off_out);
      // The kernel works on whole 16-byte vectors.  A length that is not a multiple of 16 is only
      // acceptable where the last vector ends in the block's own padding (symm_alloc pads to 16):
      // anywhere else the tail vector would overwrite the caller's elements after `count`.
      auto tail_ok = [&](const SymmBlock* b, size_t off) {
        return bytes % 16 == 0 || round_up(off + bytes, 16) == b->bytes() - I.guard_of(b);
      };
      zero_copy = sb_in && sb_out && sb_in->mc() && sb_out->mc() && (off_in % 16 == 0) && (off_out % 16 == 0) &&
                  tail_ok(sb_in, off_in) && tail_ok(sb_out, off_out);
    }
    if (algo == AllreduceAlgo::automatic) {
      // The one-shot push wins for small messages, NVLS above, the two-shot push where NVLS does not
      // apply; the sizes come from the per-rank-count table of the tuning (al_info prints it).
      if (bytes <= X.ar_oneshot_max_bytes || p == 1) algo = AllreduceAlgo::one_shot;
      // Two ranks: neither the switch nor a two-shot saves traffic (every algorithm moves S bytes each way), so
      // the one-shot push is used at every size; large messages run it pipelined (below).
      else if (p == 2 && !zero_copy) algo = AllreduceAlgo::one_shot;
      else if (nvls_ok && (zero_copy || bytes >= X.ar_nvls_min_bytes)) algo = AllreduceAlgo::nvls;
      else algo = AllreduceAlgo::two_shot;
    }
    if (algo != AllreduceAlgo::nvls) zero_copy = false;
    P.two_phase = algo == AllreduceAlgo::two_shot ? 1 : 0;
    if (algo == AllreduceAlgo::one_shot && in == wire && p > 1) {
      bool aligned = true;
      for (const RankArgs& a : ranks) aligned = aligned && a.send && (uintptr_t)a.send % 16 == 0;
      P.own_direct = aligned ? 1 : 0;
    }
  }


  // Registered buffers: reduce_scatter (send side) and allgather / alltoall / bcast (receive side) run
  // straight on them.  The decision looks at this rank's buffers only; the kernels compare protocols
  // when they enter the operation, so ranks that disagree stop with a clear error.
  bool use_window = false;
  WinParams Wp{};
  {
    const bool kind_ok = d.kind == DevColl::reduce_scatter || d.kind == DevColl::allgather ||
                         d.kind == DevColl::alltoall || d.kind == DevColl::bcast;
    const size_t slice = P.count * esz;                                    // bytes per rank slice (bcast: the vector)
    const size_t total = d.kind == DevColl::bcast ? slice : slice * (size_t)p;
    const bool wanted = d.path == CollPath::window || (d.path == CollPath::automatic && tn.window_enable && total >= X.window_min_bytes);
    if (d.path == CollPath::window && (!kind_ok || d.vector || !(in == wire && wire == out) || !window_supported(d.kind, wire, d.op)))
      throw_al_exception("the window path serves uniform reduce_scatter (f32 / f16 / bf16: sum, avg, min, max), allgather, alltoall and bcast only");
    if (kind_ok && wanted && !d.vector && p > 1 && in == wire && wire == out && P.count > 0 &&
        window_supported(d.kind, wire, d.op) && (d.kind != DevColl::reduce_scatter || slice % 16 == 0)) {
      bool ok = true;
      for (int lr = 0; ok && lr < I.nlocal; ++lr) {
        const int r = I.rank0 + lr;
        const RankArgs& a = ranks[(size_t)lr];
        const char* sb = (const char*)a.send;
        const char* rb = (const char*)a.recv;
        size_t off = 0;
        int w = -1;
        Wp.send[r] = a.send;
        Wp.recv[r] = a.recv;
        switch (d.kind) {
          case DevColl::reduce_scatter:
            // in place (the result overwrites the start of the input other ranks still read) stays staged
            ok = sb && rb && !(rb < sb + total && sb < rb + slice) && (w = find_window(sb, total, &off, lr)) >= 0;
            // Pulling slices with peer loads is slower than pushing them through staging (loads over NVLink stall
            // their threads); left to itself the library takes the window path for reduce_scatter only where
            // the switch does the reduction (multicast-bound window) and there are enough ranks for that to pay.
            if (ok && d.path == CollPath::automatic)
              ok = tn.window_multimem && I.table_host.mc[w] != nullptr && p >= tn.window_rs_min_ranks &&
                   total >= tn.window_rs_min_bytes;
            if (ok) Wp.send_desc[r] = make_desc(w, off);
            break;
          case DevColl::allgather: {
            const bool in_place = sb == rb + (size_t)r * slice;
            ok = sb && rb && (in_place || !(sb < rb + total && rb < sb + slice)) && (w = find_window(rb, total, &off, lr)) >= 0;
            if (ok) Wp.recv_desc[r] = make_desc(w, off);
            break;
          }
          case DevColl::alltoall:
            ok = sb && rb && !(sb < rb + total && rb < sb + total) && (w = find_window(rb, total, &off, lr)) >= 0;
            if (ok) Wp.recv_desc[r] = make_desc(w, off);
            break;
          case DevColl::bcast:
            ok = rb && (w = find_window(rb, total, &off, lr)) >= 0;
            if (ok) { Wp.recv_desc[r] = make_desc(w, off); Wp.send[r] = a.recv; }
            break;
          default: ok = false;
        }
      }
      use_window = ok;
    }
    if (d.path == CollPath::window && !use_window)
      throw_al_exception("the window path was requested but this rank's buffer is not registered (or the buffers overlap)");
  }

  // Large reduce_scatters of private buffers let the switch reduce: copy into the multicast-bound staging,
  // multimem.ld_reduce the own slice straight into the receive buffer.  Each GPU then receives one reduced
  // stream instead of p-1 pushed ones and reads nothing back from staging.  Eligibility depends on facts all
  // ranks share (and the kernels compare protocols anyway).
  if (d.kind == DevColl::reduce_scatter && !use_window) {
    const bool ok = !d.vector && !I.emulated && p > 2 && I.ws.mc_stage != nullptr && in == wire && wire == out &&
                    P.count > 0 && nvls_allreduce_supported(wire, d.op);
    if (d.path == CollPath::nvls && !ok)
      throw_al_exception("NVLS reduce_scatter requested but unavailable (no multicast, two ranks, vector form, or type/operator unsupported)");
    if (ok && (d.path == CollPath::nvls || (d.path == CollPath::automatic && P.count * esz * (size_t)p >= X.rs_nvls_min_bytes))) {
      NvlsParams N{};
      N.ws = I.ws;
      N.send = ranks[0].send;
      N.recv = ranks[0].recv;
      N.count = P.count;
      const size_t vec = 16 / esz;
      const size_t slot_cap_e = (half / (size_t)p) / 256 * 256 / esz;               // elements of a slice a staging half holds
      size_t chunk_e = std::max<size_t>(ceil_div(P.count, (size_t)8), (size_t{1} << 20) / esz);  // an eighth of the slice, 1 MiB at least
      chunk_e = std::min(round_up(chunk_e, vec), slot_cap_e);
      N.chunk_elems = chunk_e;
      N.chunks = ceil_div(P.count, chunk_e);
      if (N.chunks >= (1u << 24) - 2) throw_al_exception("message too large for the configured staging size");
      N.seq = P.seq;
      N.timeout_ns = P.timeout_ns;
      N.scale = P.scale;
      N.rank = I.rank0;
      const size_t work = std::min(P.count, chunk_e) * esz * (size_t)p;
      int nctas = (int)std::max<size_t>(2, std::min<size_t>((size_t)std::min(tn.max_ctas_nvls, 128), ceil_div(work, (size_t)65536)));
      I.order_after_previous(stream);
      I.stats.ops++;
      I.stats.bytes += P.count * esz * (size_t)p;
      I.stats.kernels++;
      I.stats.rs_nvls++;
      launch_nvls_reduce_scatter(N, wire, d.op, nctas, std::min(512, tn.threads_per_cta), stream);
      return;
    }
  } else if (d.path == CollPath::nvls) {
    throw_al_exception("the nvls path serves reduce_scatter (for allreduce use AllreduceAlgo::nvls)");
  }

  // Large uniform reduce_scatter / allgather / alltoall run pipelined: smaller chunks, half of the
  // grid publishing while the other half consumes.
  // The one-shot allreduce of two ranks joins them: half of the grid pushes chunk c+1 to the peer while the
  // other half reduces chunk c, so the link never waits for the reduction.
  size_t slot_e = cap_e;
  const bool ar_pipelined = d.kind == DevColl::allreduce && p == 2 && algo == AllreduceAlgo::one_shot &&
                            d.algo == AllreduceAlgo::automatic && bytes >= X.ar_pipeline_min_bytes;
  // (Real ranks also pipeline as soon as a slice does not fit one staging slot: the alternative would be
  // several chunks one after the other, each with its handshakes exposed.)
  const bool slice_exceeds_slot = !I.emulated && P.count > cap_e;
  if (((d.kind == DevColl::reduce_scatter || d.kind == DevColl::allgather || d.kind == DevColl::alltoall) && !d.vector &&
       p > 1 && !use_window && (P.count * esz >= X.pipeline_min_bytes || slice_exceeds_slot)) || ar_pipelined) {
    size_t chunk_b = std::max<size_t>(P.count * esz / 8, size_t{4} << 20);
    chunk_b = std::min(chunk_b / 256 * 256, cap_e * esz);
    if (chunk_b >= 256 && chunk_b < P.count * esz) {
      slot_e = chunk_b / esz;
      P.pipelined = 1;
      P.slot_elems = slot_e;
    }
  }

  for (int lr = 0; lr < I.nlocal; ++lr) {
    const int r = I.rank0 + lr;
    const RankArgs& a = ranks[(size_t)lr];
    P.send[r] = a.send;
    P.recv[r] = a.recv;
    CountTable& T = P.tab[r];
    if (d.vector) {
      auto fill = [&](size_t* dst, const std::vector<size_t>& src, const char* what) {
        if (src.empty()) { for (int i = 0; i < p; ++i) dst[i] = 0; return; }
        if ((int)src.size() != p) throw_al_exception(what, " must have one entry per rank");
        for (int i = 0; i < p; ++i) dst[i] = src[(size_t)i] * unit;
      };
      fill(T.send_counts, a.send_counts, "send counts");
      fill(T.send_displs, a.send_displs, "send displacements");
      fill(T.recv_counts, a.recv_counts, "receive counts");
      fill(T.recv_displs, a.recv_displs, "receive displacements");
    } else {
      for (int i = 0; i < p; ++i) {
        T.send_counts[i] = T.recv_counts[i] = d.count * unit;
        T.send_displs[i] = T.recv_displs[i] = (size_t)i * d.count * unit;
      }
    }
    size_t need = 0, chunk_unit = full_e, work = 0;
    auto mx = [&](const size_t* v) { size_t m = 0; for (int i = 0; i < p; ++i) m = std::max(m, v[i]); return m; };
    switch (d.kind) {
      case DevColl::allreduce:
        need = P.count; work = P.count;
        chunk_unit = algo == AllreduceAlgo::nvls ? full_e : (algo == AllreduceAlgo::two_shot ? (size_t)p * cap2_e : slot_e);
        break;
      case DevColl::reduce: need = P.count; chunk_unit = cap_e; work = P.count; break;
      case DevColl::bcast: need = P.count; chunk_unit = full_e; work = P.count; break;
      case DevColl::reduce_scatter: need = mx(T.recv_counts); chunk_unit = slot_e; work = need * (size_t)p; break;
      case DevColl::allgather: need = mx(T.recv_counts); chunk_unit = slot_e; work = need * (size_t)p; break;
      case DevColl::alltoall:
        need = std::max(mx(T.send_counts), mx(T.recv_counts)); chunk_unit = slot_e; work = need * (size_t)p; break;
      case DevColl::gather:
        need = r == d.root ? mx(T.recv_counts) : T.send_counts[r];
        chunk_unit = cap_e; work = r == d.root ? need * (size_t)p : need; break;
      case DevColl::scatter:
        need = r == d.root ? mx(T.send_counts) : T.recv_counts[r];
        chunk_unit = full_e; work = r == d.root ? need * (size_t)p : need; break;
      case DevColl::barrier: need = 0; break;
    }
    P.local_chunks[r] = std::max<uint64_t>(1, ceil_div(need, chunk_unit));
    if (P.local_chunks[r] >= (1u << 24) - 2) throw_al_exception("message too large for the configured staging size");
    max_work_bytes = std::max(max_work_bytes, std::min(work * esz, half));
  }

  // ---- grid ------------------------------------------------------------------------
  int threads = std::min(512, tn.threads_per_cta);
  int ctas = d.ctas > 0 ? d.ctas : (int)std::max<size_t>(1, ceil_div(max_work_bytes, (size_t)32768));
  int cap = tn.max_ctas;
  if (d.kind == DevColl::allreduce && algo == AllreduceAlgo::nvls) cap = zero_copy ? tn.max_ctas_zero_copy : tn.max_ctas_nvls;
  if (I.nlocal > 1) cap = std::min(cap, std::max(1, I.sm_count / I.nlocal));  // cooperative launch must be co-resident
  ctas = std::max(1, std::min(ctas, cap));
  if (P.pipelined) {
    // the whole budget: half publishes, half consumes; one CTA per SM at most (they wait for each other)
    ctas = std::max(2, std::min(tn.max_ctas_pipelined, I.sm_count - 4));
    if (I.nlocal > 1) ctas = std::max(2, std::min(ctas, I.sm_count / I.nlocal));
  }
  if (max_work_bytes <= 4096) threads = std::min(threads, 256);

  I.order_after_previous(stream);
  I.stats.ops++;
  I.stats.bytes += bytes ? bytes : max_work_bytes;
  I.stats.kernels++;

  if (d.kind == DevColl::allreduce && algo == AllreduceAlgo::nvls) {
    NvlsParams N{};
    N.ws = I.ws;
    N.send = ranks[0].send;
    N.recv = ranks[0].recv;
    N.count = P.count;
    N.chunks = P.local_chunks[I.rank0];
    if (!zero_copy && bytes >= X.nvls_pipeline_min_bytes) {
      // pipelined flavour: chunks of 1/16 of the message (at least 8 MiB, at most a staging half) in a ring of
      // slots laid over both halves; smaller chunks are dominated by the per-chunk handshakes
      size_t chunk_b = std::max<size_t>(bytes / 16, std::max<size_t>(tn.nvls_chunk_bytes, 65536));
      chunk_b = std::min(chunk_b / 4096 * 4096, half);
      N.chunk_elems = chunk_b / esz;
      N.chunks = ceil_div(P.count, N.chunk_elems);
      N.ring_depth = (int)std::max<size_t>(2, std::min<size_t>((size_t)kRingDepth, 2 * half / chunk_b));
      ctas = std::max(8, std::min(tn.max_ctas_nvls, 128));
    }
    N.seq = P.seq;
    N.timeout_ns = P.timeout_ns;
    N.scale = P.scale;
    N.rank = I.rank0;
    if (zero_copy) {
      N.mc_in = (const char*)sb_in->mc() + off_in;
      N.mc_out = (char*)sb_out->mc() + off_out;
      I.stats.ar_nvls_zero_copy++;
    }
    I.stats.ar_nvls++;
    launch_nvls_allreduce(N, wire, d.op, ctas, threads, stream);
    return;
  }
  if (d.kind == DevColl::allreduce) {
    if (algo == AllreduceAlgo::one_shot) I.stats.ar_one_shot++;
    else I.stats.ar_two_shot++;
  }
  if (use_window) {
    Wp.ws = I.ws;
    Wp.windows = I.table_dev;
    Wp.count = P.count;
    Wp.seq = P.seq;
    Wp.timeout_ns = P.timeout_ns;
    Wp.scale = P.scale;
    Wp.int_div = P.int_div;
    Wp.kind = P.kind;
    Wp.op = P.op;
    Wp.root = P.root;
    Wp.rank0 = I.rank0;
    // bit 0: multimem for reduce_scatter / bcast, bit 1: for allgather (only from window_multimem_ag_ranks ranks on)
    Wp.allow_multimem = tn.window_multimem ? (1 | (p >= tn.window_multimem_ag_ranks ? 2 : 0)) : 0;
    const size_t moved = P.count * esz * (d.kind == DevColl::alltoall ? (size_t)p : 1);
    int wctas = d.ctas > 0 ? d.ctas : (int)std::max<size_t>(1, std::min<size_t>(ceil_div(moved, (size_t)32768), (size_t)tn.window_ctas));
    if (I.nlocal > 1) wctas = std::max(1, std::min(wctas, I.sm_count / I.nlocal));
    I.stats.window++;
    launch_window(Wp, wire, d.op, wctas, threads, I.nlocal, stream);
    return;
  }
  // Opt-in: the pipelined schedule with the copy engine moving the data.  A rank whose buffers do
  // not qualify runs the generic kernel; the two speak the same protocol.
  if (P.pipelined && tn.bulk_pipeline && in == wire && wire == out && bulk_pipeline_supported(d.kind, wire, d.op) &&
      (P.count * esz) % 16 == 0 && (P.slot_elems * esz) % 16 == 0) {
    bool aligned = true;
    for (const RankArgs& a : ranks)
      aligned = aligned && a.send && a.recv && (uintptr_t)a.send % 16 == 0 && (uintptr_t)a.recv % 16 == 0;
    if (aligned) {
      int n_pub = tn.bulk_pub_ctas;
      int n_con = d.kind == DevColl::reduce_scatter ? std::max(1, cap / 2) : tn.bulk_con_ctas;
      if (I.nlocal > 1) {  // cooperative launch: one CTA per SM with this kernel's shared memory
        const int per_rank = std::max(2, I.sm_count / I.nlocal);
        n_pub = std::max(1, std::min(n_pub, per_rank / 2));
        n_con = std::max(1, std::min(n_con, per_rank - n_pub));
      }
      P.n_pub = n_pub;
      I.stats.bulk_pipeline++;
      launch_bulk_pipeline(P, wire, n_pub + n_con, threads, I.nlocal, stream);
      return;
    }
  }
  launch_collective(P, in, wire, out, ctas, threads, I.nlocal, stream);
}

// ---------------------------------------------------------------------------
// row exchange
// ---------------------------------------------------------------------------
void DeviceCommunicator::exchange_rows(const std::vector<RowArgs>& ranks, size_t row_bytes, size_t send_row_stride,
                                       size_t recv_row_stride, cudaStream_t stream) {
  Impl& I = *impl_;
  std::lock_guard<std::mutex> lock(I.mu);
  check_status();
  if ((int)ranks.size() != I.nlocal)
    throw_al_exception("expected arguments for ", I.nlocal, " local rank(s), got ", ranks.size());
  const int p = I.p;
  const size_t cap_b = (I.ws.half_bytes / (size_t)p) / 256 * 256;
  if (row_bytes == 0 || row_bytes > cap_b)
    throw_al_exception("exchange_rows: a row of ", row_bytes, " bytes does not fit a staging slot of ", cap_b, " bytes");
  const size_t per_chunk = cap_b / row_bytes;
  RowsParams R{};
  R.ws = I.ws;
  R.row_bytes = row_bytes;
  R.send_row_stride = send_row_stride;
  R.recv_row_stride = recv_row_stride;
  R.seq = ++I.seq;
  R.timeout_ns = I.timeout_ns;
  R.rank0 = I.rank0;
  size_t most_rows = 0, total_rows = 0;
  for (int lr = 0; lr < I.nlocal; ++lr) {
    const int r = I.rank0 + lr;
    const RowArgs& a = ranks[(size_t)lr];
    auto fill = [&](size_t* dst, const std::vector<size_t>& src, const char* what) {
      if ((int)src.size() != p) throw_al_exception("exchange_rows: ", what, " must have one entry per rank");
      for (int i = 0; i < p; ++i) dst[i] = src[(size_t)i];
    };
    RowTable& T = R.tab[r];
    fill(T.send_rows, a.send_rows, "send_rows");
    fill(T.send_first, a.send_first, "send_first");
    fill(T.send_peer_off, a.send_peer_off, "send_peer_off");
    fill(T.recv_rows, a.recv_rows, "recv_rows");
    fill(T.recv_first, a.recv_first, "recv_first");
    fill(T.recv_peer_off, a.recv_peer_off, "recv_peer_off");
    R.send[r] = a.send;
    R.recv[r] = a.recv;
    R.send_idx[r] = a.send_idx;
    R.recv_idx[r] = a.recv_idx;
    size_t mx = 0;
    for (int i = 0; i < p; ++i) {
      mx = std::max(mx, std::max(T.send_rows[i], T.recv_rows[i]));
      total_rows += T.send_rows[i];
    }
    most_rows = std::max(most_rows, mx);
    R.local_chunks[r] = std::max<uint64_t>(1, ceil_div(mx, per_chunk));
    if (R.local_chunks[r] >= (1u << 24) - 2) throw_al_exception("exchange_rows: too many rows for the configured staging size");
  }
  const size_t work = std::min(total_rows / (size_t)I.nlocal, per_chunk * (size_t)p) * row_bytes;
  int ctas = (int)std::max<size_t>(1, std::min<size_t>(ceil_div(work, (size_t)65536), (size_t)tuning().max_ctas));
  if (I.nlocal > 1) ctas = std::max(1, std::min(ctas, I.sm_count / I.nlocal));
  const int threads = work <= 16384 ? 128 : 512;
  I.order_after_previous(stream);
  I.stats.ops++;
  I.stats.bytes += total_rows * row_bytes;
  I.stats.kernels++;
  I.stats.rows++;
  launch_rows(R, ctas, threads, I.nlocal, stream);
}

// ---------------------------------------------------------------------------
// point-to-point
// ---------------------------------------------------------------------------
void DeviceCommunicator::p2p(const std::vector<P2PDesc>& items_in, cudaStream_t stream) {
  Impl& I = *impl_;
  std::lock_guard<std::mutex> lock(I.mu);
  check_status();
  if (items_in.empty()) return;
  const size_t slot = I.ws.mbox_slot_bytes;
  // Transfers of the same (owner, peer, direction) must not share a launch:
  // their pieces are numbered consecutively and have to land in order.
  std::vector<char> placed(items_in.size(), 0);
  size_t remaining = items_in.size();
  I.order_after_previous(stream);
  // A buffer that is both sent and received by the same rank (in-place SendRecv /
  // MultiSendRecv) is sent from a stream-ordered temporary copy, so that arriving
  // data cannot overwrite bytes that have not left yet.
  std::vector<P2PDesc> staged(items_in);
  std::vector<void*> temps;
  for (auto& s : staged) {
    if (!s.is_send || s.bytes == 0) continue;
    for (const auto& r : items_in) {
      if (r.is_send || r.bytes == 0 || r.owner != s.owner) continue;
      const char* sb = (const char*)s.sbuf;
      const char* rb = (const char*)r.rbuf;
      if (sb < rb + r.bytes && rb < sb + s.bytes) {
        void* t = nullptr;
        AL_CHECK_CUDA(cudaMallocAsync(&t, s.bytes, stream));
        AL_CHECK_CUDA(cudaMemcpyAsync(t, s.sbuf, s.bytes, cudaMemcpyDeviceToDevice, stream));
        s.sbuf = t;
        temps.push_back(t);
        break;
      }
    }
  }
  const std::vector<P2PDesc>& items = staged;
  while (remaining) {
    P2PParams P{};
    P.ws = I.ws;
    P.timeout_ns = I.timeout_ns;
    P.windows = I.table_dev;
    P.rendezvous_bytes = tuning().p2p_rendezvous_bytes ? tuning().p2p_rendezvous_bytes : ~size_t{0};
    P.ll_bytes = std::min(tuning().p2p_ll_max_bytes, I.ws.p2p_ll_slot_bytes / 2);
    P.launch = ++I.p2p_launches;
    size_t biggest_direct = 0;
    std::vector<uint64_t> used;  // keys taken in this launch
    size_t biggest = 0;
    for (size_t i = 0; i < items.size() && P.nitems < P2PParams::kMaxItems; ++i) {
      if (placed[i]) continue;
      const P2PDesc& it = items[i];
      const int owner = I.emulated ? it.owner : I.rank0;
      if (owner < I.rank0 || owner >= I.rank0 + I.nlocal) throw_al_exception("p2p: owner rank ", owner, " is not local");
      if (it.peer < 0 || it.peer >= I.p) throw_al_exception("p2p: peer ", it.peer, " out of range");
      const uint64_t key = ((uint64_t)owner << 32) | ((uint64_t)it.peer << 1) | (it.is_send ? 1u : 0u);
      if (std::find(used.begin(), used.end(), key) != used.end()) continue;
      used.push_back(key);
      const int k = P.nitems++;
      P.sbuf[k] = it.sbuf;
      P.rbuf[k] = it.rbuf;
      P.bytes[k] = it.bytes;
      P.peer[k] = it.peer;
      P.is_send[k] = it.is_send ? 1 : 0;
      P.owner[k] = owner;
      if (!it.is_send && it.bytes >= P.rendezvous_bytes) {
        // a registered receive buffer is announced to the sender, which then stores straight into it
        size_t off = 0;
        const int w = find_window(it.rbuf, it.bytes, &off, owner - I.rank0);
        if (w >= 0) P.rdesc[k] = make_desc(w, off);
      }
      if (it.bytes >= P.rendezvous_bytes) biggest_direct = std::max(biggest_direct, it.bytes);
      auto& ctr = it.is_send ? I.p2p_sent : I.p2p_recvd;
      uint64_t& c = ctr[(size_t)(owner - I.rank0) * (size_t)I.p + (size_t)it.peer];
      P.base[k] = c;
      c += std::max<size_t>(1, ceil_div(it.bytes, slot));
      biggest = std::max(biggest, it.bytes);
      placed[i] = 1;
      --remaining;
      I.stats.bytes += it.bytes;
    }
    // CTAs per transfer: one per 64 KiB of a mailbox piece - or of the whole message where it may go straight
    // into a registered buffer - up to the tuning's cap.
    int per = (int)std::max<size_t>(1, std::min<size_t>(ceil_div(std::max(std::min(biggest, slot), biggest_direct), (size_t)65536), (size_t)tuning().p2p_max_ctas));
    if (I.nlocal > 1) per = std::max(1, std::min(per, I.sm_count / P.nitems));
    else per = std::max(1, std::min(per, 2 * I.sm_count / P.nitems));  // waiting CTAs must all be resident
    P.ctas_per_item = per;
    I.stats.ops++;
    I.stats.kernels++;
    launch_p2p(P, 512, I.nlocal > 1 ? 1 : 0, stream);
  }
  for (void* t : temps) AL_CHECK_CUDA(cudaFreeAsync(t, stream));
}

// ---------------------------------------------------------------------------
// symmetric user memory
// ---------------------------------------------------------------------------
namespace {
constexpr size_t kGuardBytes = 4096;
constexpr int kGuardByte = 0xA5;
}  // namespace

void* DeviceCommunicator::symm_alloc(size_t bytes) {
  Impl& I = *impl_;
  std::unique_ptr<SymmBlock> b;
  const size_t padded = round_up(std::max<size_t>(bytes, 16), 16);
  // Guard mode (AL_DEBUG_GUARD=1): a region of a known byte pattern before and after the user's part of
  // every symmetric block; check_guards() (also run by symm_free) reports a kernel - of this library or of
  // the caller - that wrote outside the buffer.  The stand-in for a memory checker on the device.
  const size_t guard = tuning().debug_guard ? kGuardBytes : 0;
  if (I.emulated) b = SymmBlock::create_emulated(I.p, padded + 2 * guard);
  else b = SymmBlock::create(group_, padded + 2 * guard, true);
  if (guard) {
    for (int lr = 0; lr < I.nlocal; ++lr) {
      char* base = (char*)b->peer(I.rank0 + lr);
      AL_CHECK_CUDA(cudaMemset(base, kGuardByte, guard));
      AL_CHECK_CUDA(cudaMemset(base + guard + padded, kGuardByte, guard));
    }
    AL_CHECK_CUDA(cudaDeviceSynchronize());
    if (!I.emulated) group_.barrier();  // nobody uses the block before every rank's guards are in place
  }
  void* ptr = (char*)b->peer(I.emulated ? 0 : I.rank0) + guard;
  std::lock_guard<std::mutex> lock(I.mu);
  I.add_block_window(b.get());
  I.user_blocks.push_back(std::move(b));
  I.user_guard.push_back(guard);
  return ptr;
}

void DeviceCommunicator::check_guards() const {
  const Impl& I = *impl_;
  AL_CHECK_CUDA(cudaDeviceSynchronize());
  std::vector<unsigned char> h(kGuardBytes);
  for (size_t i = 0; i < I.user_blocks.size(); ++i) {
    const size_t guard = I.user_guard[i];
    if (!guard) continue;
    const SymmBlock* b = I.user_blocks[i].get();
    for (int lr = 0; lr < I.nlocal; ++lr) {
      const char* base = (const char*)b->peer(I.rank0 + lr);
      for (int side = 0; side < 2; ++side) {
        const char* g = side == 0 ? base : base + b->bytes() - guard;
        AL_CHECK_CUDA(cudaMemcpy(h.data(), g, guard, cudaMemcpyDeviceToHost));
        for (size_t k = 0; k < guard; ++k) {
          if (h[k] == (unsigned char)kGuardByte) continue;
          const long dist = side == 0 ? (long)k - (long)guard : (long)k;
          throw_al_exception("guard region of symmetric block ", i, " (rank ", I.rank0 + lr, ") was overwritten: byte at ",
                             side == 0 ? "offset " : "offset end+", dist, side == 0 ? " before the buffer" : " after the buffer",
                             " holds ", (int)h[k]);
        }
      }
    }
  }
}

void DeviceCommunicator::symm_free(void* ptr) {
  Impl& I = *impl_;
  std::unique_ptr<SymmBlock> victim;
  bool guarded = false;
  {
    std::lock_guard<std::mutex> lock(I.mu);
    for (size_t i = 0; i < I.user_blocks.size(); ++i) {
      if ((char*)I.user_blocks[i]->peer(I.emulated ? 0 : I.rank0) + I.user_guard[i] == ptr) {
        if (I.user_guard[i]) {
          guarded = true;
          break;
        }
        victim = std::move(I.user_blocks[i]);
        I.user_blocks.erase(I.user_blocks.begin() + (long)i);
        I.user_guard.erase(I.user_guard.begin() + (long)i);
        break;
      }
    }
  }
  if (guarded) {
    check_guards();  // throws if anything wrote outside a guarded buffer; the block is then kept for inspection
    std::lock_guard<std::mutex> lock(I.mu);
    for (size_t i = 0; i < I.user_blocks.size(); ++i) {
      if ((char*)I.user_blocks[i]->peer(I.emulated ? 0 : I.rank0) + I.user_guard[i] == ptr) {
        victim = std::move(I.user_blocks[i]);
        I.user_blocks.erase(I.user_blocks.begin() + (long)i);
        I.user_guard.erase(I.user_guard.begin() + (long)i);
        break;
      }
    }
  }
  if (!victim) throw_al_exception("symm_free: pointer was not returned by symm_alloc of this communicator");
  AL_CHECK_CUDA(cudaDeviceSynchronize());
  if (!I.emulated) group_.barrier();  // nobody may still be addressing the block
  {
    std::lock_guard<std::mutex> lock(I.mu);
    for (int w = 0; w < kMaxWindows; ++w)
      if (I.windows[w].used && I.windows[w].block == victim.get()) I.clear_window(w);
    I.push_table();
  }
  victim.reset();
}

const SymmBlock* DeviceCommunicator::find_symm(const void* ptr, size_t bytes, size_t* offset) const {
  const Impl& I = *impl_;
  const int me = I.emulated ? 0 : I.rank0;
  for (const auto& b : I.user_blocks) {
    const char* base = (const char*)b->peer(me);
    if ((const char*)ptr >= base && (const char*)ptr + bytes <= base + b->bytes()) {
      if (offset) *offset = (size_t)((const char*)ptr - base);
      return b.get();
    }
  }
  return nullptr;
}

int DeviceCommunicator::symm_index(const void* ptr) const {
  const Impl& I = *impl_;
  const int me = I.emulated ? 0 : I.rank0;
  for (size_t i = 0; i < I.user_blocks.size(); ++i) {
    const char* base = (const char*)I.user_blocks[i]->peer(me);
    if ((const char*)ptr >= base && (const char*)ptr < base + I.user_blocks[i]->bytes()) return (int)i;
  }
  return -1;
}

void* DeviceCommunicator::symm_peer_ptr(int index, int peer, size_t offset) const {
  const Impl& I = *impl_;
  if (index < 0 || (size_t)index >= I.user_blocks.size() || peer < 0 || peer >= I.p) return nullptr;
  if (offset >= I.user_blocks[(size_t)index]->bytes()) return nullptr;
  return (char*)I.user_blocks[(size_t)index]->peer(peer) + offset;
}

// ---------------------------------------------------------------------------
// registered buffers
// ---------------------------------------------------------------------------
namespace {
struct RegMsg {
  int kind;            // 0: cannot be shared, 1: inside symmetric block `block_index`, 2: CUDA IPC handle
  int block_index;
  size_t offset;       // of the buffer inside the block / the IPC allocation
  size_t bytes;
  cudaIpcMemHandle_t handle;
};
}  // namespace

int DeviceCommunicator::register_buffer(void* ptr, size_t bytes) {
  Impl& I = *impl_;
  if (I.emulated) throw_al_exception("register_buffer: use register_buffers_emulated on an emulated communicator");
  check_status();
  RegMsg mine{};
  mine.bytes = bytes;
  size_t off = 0;
  if (ptr && bytes) {
    if (find_symm(ptr, bytes, &off)) {
      mine.kind = 1;
      mine.block_index = symm_index(ptr);
      mine.offset = off;
    } else {
      CUdeviceptr base = 0;
      size_t size = 0;
      const auto& dr = cuda::drv();
      if (dr.MemGetAddressRange && dr.MemGetAddressRange(&base, &size, (CUdeviceptr)ptr) == CUDA_SUCCESS &&
          cudaIpcGetMemHandle(&mine.handle, (void*)base) == cudaSuccess) {
        mine.kind = 2;
        mine.offset = (size_t)((CUdeviceptr)ptr - base);
      } else {
        (void)cudaGetLastError();  // memory that CUDA IPC cannot export (e.g. a VMM allocation): not registered
      }
    }
  }
  const int p = I.p;
  std::vector<RegMsg> all((size_t)p);
  group_.allgather(&mine, all.data(), sizeof(RegMsg));
  bool ok = true;
  for (const auto& m : all) ok = ok && m.kind != 0;
  std::lock_guard<std::mutex> lock(I.mu);
  const int w = ok ? I.free_window() : -1;
  if (w < 0) return -1;  // consistent on every rank: same messages, same table occupancy
  Impl::Window& W = I.windows[w];
  bool same_block = true;
  for (int r = 0; r < p; ++r) {
    const RegMsg& m = all[(size_t)r];
    same_block = same_block && m.kind == 1 && m.block_index == all[0].block_index && m.offset == all[0].offset;
    char* addr = nullptr;
    if (r == I.rank0) {
      addr = (char*)ptr;
    } else if (m.kind == 1) {
      addr = (char*)symm_peer_ptr(m.block_index, r, m.offset);
    } else {
      void* base = nullptr;
      if (cudaIpcOpenMemHandle(&base, m.handle, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess) {
        W.opened.push_back(base);
        addr = (char*)base + m.offset;
      } else {
        (void)cudaGetLastError();
      }
    }
    I.table_host.peer[w][r] = addr;
    I.table_host.bytes[w][r] = m.bytes;
  }
  // A mapping that failed on any rank voids the window on every rank.
  int good = 1;
  for (int r = 0; r < p; ++r) good = good && I.table_host.peer[w][r] != nullptr;
  std::vector<int> goods((size_t)p);
  group_.allgather(&good, goods.data(), sizeof(int));
  for (int g : goods) good = good && g;
  if (!good) {
    I.clear_window(w);
    return -1;
  }
  W.used = true;
  W.local[I.rank0] = ptr;
  if (same_block && all[0].kind == 1) {
    const SymmBlock* b = I.user_blocks[(size_t)all[0].block_index].get();
    if (b->mc()) I.table_host.mc[w] = (char*)b->mc() + all[0].offset;
  }
  I.push_table();
  return w;
}

int DeviceCommunicator::register_buffers_emulated(const std::vector<void*>& ptrs, size_t bytes) {
  Impl& I = *impl_;
  if (!I.emulated) throw_al_exception("register_buffers_emulated: not an emulated communicator");
  if ((int)ptrs.size() != I.p) throw_al_exception("register_buffers_emulated: one buffer per rank expected");
  std::lock_guard<std::mutex> lock(I.mu);
  const int w = I.free_window();
  if (w < 0) return -1;
  Impl::Window& W = I.windows[w];
  W.used = true;
  for (int r = 0; r < I.p; ++r) {
    W.local[r] = ptrs[(size_t)r];
    I.table_host.peer[w][r] = (char*)ptrs[(size_t)r];
    I.table_host.bytes[w][r] = bytes;
  }
  I.push_table();
  return w;
}

void DeviceCommunicator::unregister_buffer(void* ptr) {
  Impl& I = *impl_;
  int w = -1;
  {
    std::lock_guard<std::mutex> lock(I.mu);
    for (int i = 0; i < kMaxWindows && w < 0; ++i)
      if (I.windows[i].used && !I.windows[i].block && I.windows[i].local[I.emulated ? 0 : I.rank0] == ptr) w = i;
  }
  // Collective: every rank drains its work and all meet before any mapping goes away.
  AL_CHECK_CUDA(cudaDeviceSynchronize());
  if (!I.emulated) group_.barrier();
  if (w < 0) return;  // was never registered (registration may have been refused on every rank)
  std::lock_guard<std::mutex> lock(I.mu);
  I.clear_window(w);
  I.push_table();
}

int DeviceCommunicator::find_window(const void* ptr, size_t bytes, size_t* offset, int local_rank) const {
  const Impl& I = *impl_;
  const int r = I.rank0 + local_rank;
  for (int w = 0; w < kMaxWindows; ++w) {
    if (!I.windows[w].used) continue;
    const char* base = (const char*)I.windows[w].local[r];
    if (!base) continue;
    if ((const char*)ptr >= base && (const char*)ptr + bytes <= base + I.table_host.bytes[w][r]) {
      if (offset) *offset = (size_t)((const char*)ptr - base);
      return w;
    }
  }
  return -1;
}

uint64_t DeviceCommunicator::wait_timeout_ns() const { return impl_->timeout_ns; }

}  // namespace Al
