// Unit tests of the host runtime pieces that need no second rank: integer
// helpers, the lock-free queues (with a concurrent stress), the caching
// allocator, the resource pool, the progress engine's ordering / concurrency
// rules, tracing, host reductions and the life cycle.  The reference has no
// unit tests for these components; they are covered here because every backend
// stands on them.
#include <algorithm>
#include <cmath>
#include <sstream>
#include <atomic>
#include <cstdio>
#include <mutex>
#include <thread>

#include "Al.hpp"
#include "al/host/reduce.hpp"
#include "al/mempool.hpp"
#include "al/util/caching_allocator.hpp"
#include "al/util/mpsc_queue.hpp"
#include "al/util/resource_pool.hpp"
#include "al/util/spsc_queue.hpp"
#include "../kernels/bulk_tiles.cuh"
#include <cstring>
#include <random>

using namespace Al;
using namespace Al::internal;

static int g_fail = 0;
#define CHECK(c) do { if (!(c)) { fprintf(stderr, "FAIL %s:%d: %s\n", __FILE__, __LINE__, #c); ++g_fail; } } while (0)

static void test_meta() {
  CHECK(is_pow2(1) && is_pow2(64) && !is_pow2(0) && !is_pow2(48));
  CHECK(floor_log2(1) == 0 && floor_log2(1023) == 9 && ceil_log2(1025) == 11 && ceil_log2(1024) == 10);
  CHECK(next_highest_pow2(17) == 32 && next_highest_pow2(32) == 32);
  CHECK(num_pow2s_between(1, 64) == 7 && num_pow2s_between(3, 5) == 1);
  auto a = pow2_ar<4>(8);
  CHECK(a[0] == 8 && a[3] == 64);
  std::vector<size_t> v{3, 0, 5};
  auto ps = excl_prefix_sum(v);
  CHECK(ps[0] == 0 && ps[1] == 3 && ps[2] == 3);
}

static void test_spsc() {
  SPSCQueue<int*> q(8);
  int vals[16];
  for (int i = 0; i < 8; ++i) CHECK(q.try_push(&vals[i]));
  CHECK(!q.try_push(&vals[8]));
  int* out = nullptr;
  CHECK(q.peek(out) && out == &vals[0]);
  q.pop_always();
  CHECK(q.pop(out) && out == &vals[1]);
  // concurrent: order and completeness
  SPSCQueue<size_t> big(1024);
  const size_t N = 2000000;
  std::thread prod([&] { for (size_t i = 1; i <= N;) if (big.try_push(i)) ++i; });
  size_t expect = 1, got;
  while (expect <= N) if (big.pop(got)) { CHECK(got == expect); ++expect; }
  prod.join();
}

static void test_mpsc() {
  MPSCQueue<size_t> q(4096);
  const int P = 4;
  const size_t N = 300000;
  std::vector<std::thread> prods;
  for (int t = 0; t < P; ++t)
    prods.emplace_back([&, t] { for (size_t i = 0; i < N;) if (q.try_push((size_t)t * N + i)) ++i; });
  std::vector<size_t> next(P, 0);
  size_t total = 0, v;
  while (total < P * N) {
    if (q.pop(v)) {
      const size_t t = v / N, i = v % N;
      CHECK(i == next[t]);  // per-producer order is preserved
      next[t] = i + 1;
      ++total;
    }
  }
  for (auto& th : prods) th.join();
  CHECK(!q.pop(v));
}

struct CountingRaw {
  static int live;
  void* allocate(size_t b) { ++live; return malloc(b); }
  void deallocate(void* p, size_t) { --live; free(p); }
};
int CountingRaw::live = 0;

static void test_allocator() {
  CHECK(SizeClasses::bin_size(SizeClasses::bin_of(100)) >= 100);
  for (size_t s : {1ul, 64ul, 65ul, 1000ul, 4097ul, 1000000ul, (1ul << 28)})
    CHECK(SizeClasses::bin_size(SizeClasses::bin_of(s)) >= s && SizeClasses::bin_size(SizeClasses::bin_of(s)) < s * 5 / 4 + 65);
  CachingAllocator<CountingRaw> a;
  void* p = a.allocate(1000);
  a.release(p);
  void* q = a.allocate(900);  // same class: must be served from the cache
  CHECK(q == p && a.hits() == 1);
  void* huge = a.allocate((1ul << 28) + 5);
  a.release(huge);  // above the largest class: returned immediately
  a.release(q);
  CHECK(CountingRaw::live == 1);
  a.clear();
  CHECK(CountingRaw::live == 0);
  bool threw = false;
  try { int x; a.release(&x); } catch (const al_exception&) { threw = true; }
  CHECK(threw);
  int* hp = mempool.allocate<MemoryType::HOST, int>(100);
  hp[99] = 7;
  mempool.release<MemoryType::HOST>(hp);
}

struct IntFactory {
  int next = 0;
  int create() { return ++next; }
  void destroy(int) {}
};

static void test_pool() {
  LockedResourcePool<int, IntFactory> pool;
  pool.preallocate(3);
  CHECK(pool.idle() == 3);
  int a = pool.get(), b = pool.get(), c = pool.get(), d = pool.get();
  CHECK(pool.idle() == 0 && d == 4 && a != b && b != c);
  pool.release(a);
  CHECK(pool.get() == a);
  pool.clear();
}

// A state that records when it ran and finishes after a number of steps.
// Completion log shared between the engine thread (writer) and the test (reader).
struct ProbeLog {
  void push(int id) { std::lock_guard<std::mutex> g(m); ids.push_back(id); }
  size_t size() { std::lock_guard<std::mutex> g(m); return ids.size(); }
  int at(size_t i) { std::lock_guard<std::mutex> g(m); return ids[i]; }
  void clear() { std::lock_guard<std::mutex> g(m); ids.clear(); }
  std::mutex m;
  std::vector<int> ids;
};

struct ProbeState : AlState {
  ProbeState(const void* key, int id, int steps, ProbeLog* log, std::atomic<int>* running, std::atomic<int>* peak,
             RunType rt = RunType::bounded, bool advance = false)
      : key_(key), id_(id), left_(steps), log_(log), running_(running), peak_(peak), rt_(rt), adv_(advance) {}
  void start() override {
    int r = ++*running_;
    int p = peak_->load();
    while (r > p && !peak_->compare_exchange_weak(p, r)) {}
  }
  PEAction step() override {
    if (adv_ && !advanced_) { advanced_ = true; return PEAction::advance; }
    if (--left_ > 0) return PEAction::cont;
    log_->push(id_);
    --*running_;
    return PEAction::complete;
  }
  const void* get_compute_stream() const override { return key_; }
  RunType get_run_type() const override { return rt_; }
  const char* get_name() const override { return "Probe"; }
  const void* key_;
  int id_, left_;
  ProbeLog* log_;
  std::atomic<int>*running_, *peak_;
  RunType rt_;
  bool adv_, advanced_ = false;
};

static void test_progress_engine() {
  ProgressEngine pe;
  ProbeLog log;
  std::atomic<int> running{0}, peak{0};
  int k1, k2;
  // Same stream: bounded states beyond the limit wait; completion order of equal-length states is FIFO.
  for (int i = 0; i < 12; ++i) pe.enqueue(new ProbeState(&k1, i, 200, &log, &running, &peak));
  while (pe.in_flight() || log.size() < 12) std::this_thread::yield();
  CHECK(peak.load() <= std::max(1, tuning().pe_num_concurrent_ops));
  for (int i = 0; i < 12; ++i) CHECK(log.at((size_t)i) == i);
  // Unbounded states are all admitted at once.
  log.clear(); peak = 0;
  for (int i = 0; i < 10; ++i) pe.enqueue(new ProbeState(&k2, i, 2000, &log, &running, &peak, RunType::unbounded));
  while (log.size() < 10) std::this_thread::yield();
  CHECK(peak.load() == 10);
  // Pipeline: states advance to stage 1 in order.
  log.clear();
  for (int i = 0; i < 4; ++i) pe.enqueue(new ProbeState(&k1, i, 10 * (4 - i), &log, &running, &peak, RunType::bounded, true));
  while (log.size() < 4) std::this_thread::yield();
  std::ostringstream ss;
  pe.dump_state(ss);
  CHECK(ss.str().find("Progress engine") != std::string::npos);
  pe.stop();
  CHECK(!pe.is_running());
}

// Several user threads hand their first state to an engine that is not running yet:
// exactly one of them may create the thread, the others wait for it.
static void test_progress_engine_concurrent_start() {
  for (int round = 0; round < 20; ++round) {
    ProgressEngine pe;
    ProbeLog log;
    std::atomic<int> running{0}, peak{0}, go{0};
    int keys[4];
    std::vector<std::thread> th;
    for (int t = 0; t < 4; ++t)
      th.emplace_back([&, t] {
        while (!go.load()) std::this_thread::yield();
        for (int i = 0; i < 8; ++i) pe.enqueue(new ProbeState(&keys[t], t * 8 + i, 5, &log, &running, &peak));
      });
    go = 1;
    for (auto& x : th) x.join();
    while (log.size() < 32) std::this_thread::yield();
    pe.stop();
    CHECK(log.size() == 32);
  }
}

// Ordering domains come and go (communicators are created and destroyed): released slots are reused,
// so more than AL_PE_NUM_STREAMS domains can be served over the life of the engine.
static void test_progress_engine_slot_reuse() {
  ProgressEngine pe;
  ProbeLog log;
  std::atomic<int> running{0}, peak{0};
  std::vector<int> keys(3 * AL_PE_NUM_STREAMS);
  for (size_t k = 0; k < keys.size(); ++k) {
    pe.enqueue(new ProbeState(&keys[k], (int)k, 3, &log, &running, &peak));
    while (log.size() < k + 1) std::this_thread::yield();
    pe.release_key(&keys[k]);
  }
  CHECK(log.size() == keys.size());
  // Without release the table fills up and says so.
  bool threw = false;
  try {
    for (size_t k = 0; k < keys.size(); ++k) pe.enqueue(new ProbeState(&keys[k], (int)k, 1, &log, &running, &peak));
  } catch (const Al::al_exception&) {
    threw = true;
  }
  CHECK(threw);
  while (pe.in_flight()) std::this_thread::yield();
  pe.stop();
}

static void test_reduce_and_halves() {
  using namespace Al::internal::host;
  for (float f : {0.f, 1.f, -2.5f, 65504.f, 6.1e-5f, 1e-7f, 0.333f}) {
    const float back = half_to_float(float_to_half(f));
    CHECK(std::fabs(back - f) <= std::fabs(f) * 1e-3f + 1e-7f);
    const float b2 = bf16_to_float(float_to_bf16(f));
    CHECK(std::fabs(b2 - f) <= std::fabs(f) * 8e-3f + 1e-30f);
  }
  CHECK(float_to_half(1e6f) == 0x7c00);
  int a[4] = {1, 2, 3, 4}, b[4] = {4, 3, 2, 1}, out[4];
  const void* srcs[2] = {a, b};
  reduce_multi(DType::i32, ReductionOperator::max, out, srcs, 2, 4);
  CHECK(out[0] == 4 && out[1] == 3 && out[2] == 3 && out[3] == 4);
  reduce_multi(DType::i32, ReductionOperator::bxor, out, srcs, 2, 4);
  CHECK(out[0] == 5 && out[3] == 5);
  reduce_multi(DType::i32, ReductionOperator::avg, out, srcs, 2, 4);
  CHECK(out[0] == 2 && out[1] == 2);
  CHECK(!Al::internal::host::reduction_supported(DType::f32, ReductionOperator::band));
  bool threw = false;
  float fa[1] = {1}, fo[1];
  const void* fs[1] = {fa};
  try { reduce_multi(DType::f32, ReductionOperator::bor, fo, fs, 1, 1); } catch (const al_exception&) { threw = true; }
  CHECK(threw);
}

static void test_lifecycle_and_trace() {
  CHECK(!Initialized());
  Initialize();
  Initialize();  // idempotent
  CHECK(Initialized());
  trace::enable(true);
  {
    HostCommunicator comm;
    CHECK(comm.size() == 1 && comm.rank() == 0);
    float x[8] = {1, 2, 3, 4, 5, 6, 7, 8};
    Allreduce<HostBackend>(x, 8, ReductionOperator::sum, comm);
    CHECK(x[7] == 8);
    HostBackend::req_type req;
    NonblockingAllreduce<HostBackend>(x, 8, ReductionOperator::sum, comm, req);
    Wait<HostBackend>(req);
    CHECK(req == nullptr);
    NonblockingBarrier<HostBackend>(comm, req);
    while (!Test<HostBackend>(req)) {}
    CHECK(Test<HostBackend>(req));  // a null request tests as complete
    float y[4] = {9, 9, 9, 9};
    SendRecv<HostBackend>(y, 4, 0, 0, comm);  // self exchange in place
    CHECK(y[0] == 9);
  }
  auto lines = trace::snapshot();
  bool saw = false, saw_pe = false;
  for (auto& l : lines) {
    if (l.find("HostBackend float allreduce 0 1") != std::string::npos) saw = true;
    if (l.find("PE START") != std::string::npos) saw_pe = true;
  }
  CHECK(saw && saw_pe);
  trace::enable(false);
  trace::clear();
  Finalize();
  Finalize();
  CHECK(!Initialized());
  bool threw = false;
  try { HostCommunicator c; } catch (const al_exception&) { threw = true; }
  CHECK(threw);
}

// The tile plans of the bulk-copy kernels, executed on host memory: every byte must arrive exactly
// once at the place the collective defines, every transfer must satisfy the copy engine's 16-byte
// rules and stay inside its staging slot.
static void test_bulk_tile_plans() {
  using namespace Al::internal::device::plan;
  using Bytes = std::vector<unsigned char>;
  std::minstd_rand rng(7);
  const size_t tile = 64;  // the plans are parametric in the tile size; a small one gives many tiles
  auto fill = [&](Bytes& b, int r) { for (size_t i = 0; i < b.size(); ++i) b[i] = (unsigned char)((i * 131 + (size_t)r * 29 + (i >> 8)) & 0xff); };
  auto ok16 = [&](const Move& m) { return m.bytes > 0 && m.bytes % 16 == 0 && m.src % 16 == 0 && m.dst % 16 == 0 && m.bytes <= tile; };
  for (int p : {2, 3, 4, 8}) {
    for (int trial = 0; trial < 8; ++trial) {
      const size_t slice = 16 * (1 + rng() % 300);
      const size_t cap = 256 * (1 + rng() % 4);
      const size_t slot = 16 * (1 + rng() % (cap / 16));
      const unsigned n_pub = 1 + rng() % 5, n_con = 1 + rng() % 5;
      const uint64_t G = (slice + slot - 1) / slot;
      // ---- staged allgather: send = one slice, receive = p slices ----------------------------------
      {
        std::vector<Bytes> send((size_t)p, Bytes(slice)), recv((size_t)p, Bytes(slice * (size_t)p, 0));
        std::vector<std::vector<int>> hits((size_t)p, std::vector<int>(slice * (size_t)p, 0));
        std::vector<Bytes> stage((size_t)p, Bytes(2 * cap * (size_t)p, 0xEE));
        for (int r = 0; r < p; ++r) fill(send[(size_t)r], r);
        for (uint64_t c = 0; c < G; ++c) {
          const size_t half = (c & 1) * cap * (size_t)p;
          for (int r = 0; r < p; ++r)
            for (unsigned part = 0; part < n_pub; ++part) {
              const Share sh = share_of(slice, slot, c, part, n_pub, tile);
              for (size_t k = 0; k < sh.tiles; ++k) {
                const Move m = ag_publish(sh, k, r, cap, tile);
                CHECK(ok16(m) && m.peer == -1 && m.src + m.bytes <= slice);
                CHECK(m.dst >= (size_t)r * cap && m.dst + m.bytes <= (size_t)(r + 1) * cap);
                for (int d = 0; d < p; ++d) memcpy(&stage[(size_t)d][half + m.dst], &send[(size_t)r][m.src], m.bytes);
              }
            }
          for (int r = 0; r < p; ++r)
            for (unsigned part = 0; part < n_con; ++part) {
              const Share sh = share_of(slice, slot, c, part, n_con, tile);
              for (size_t t = 0; t < fan_tiles(sh, p); ++t) {
                const Move m = gather_consume(sh, t, p, slice, cap, tile);
                CHECK(ok16(m) && m.dst + m.bytes <= slice * (size_t)p);
                memcpy(&recv[(size_t)r][m.dst], &stage[(size_t)r][half + m.src], m.bytes);
                for (size_t i = 0; i < m.bytes; ++i) hits[(size_t)r][m.dst + i]++;
              }
            }
        }
        for (int r = 0; r < p; ++r) {
          bool same = true, once = true;
          for (int q = 0; q < p; ++q) same = same && memcmp(&recv[(size_t)r][(size_t)q * slice], send[(size_t)q].data(), slice) == 0;
          for (int h : hits[(size_t)r]) once = once && h == 1;
          CHECK(same && once);
        }
      }
      // ---- staged alltoall (and the publish half of reduce_scatter): send = p slices ------------------
      {
        std::vector<Bytes> send((size_t)p, Bytes(slice * (size_t)p)), recv((size_t)p, Bytes(slice * (size_t)p, 0));
        std::vector<Bytes> stage((size_t)p, Bytes(2 * cap * (size_t)p, 0xEE));
        for (int r = 0; r < p; ++r) fill(send[(size_t)r], r + 40);
        for (uint64_t c = 0; c < G; ++c) {
          const size_t half = (c & 1) * cap * (size_t)p;
          for (int r = 0; r < p; ++r)
            for (unsigned part = 0; part < n_pub; ++part) {
              const Share sh = share_of(slice, slot, c, part, n_pub, tile);
              for (size_t t = 0; t < fan_tiles(sh, p); ++t) {
                const Move m = scatter_publish(sh, t, r, p, slice, cap, tile);
                CHECK(ok16(m) && m.peer >= 0 && m.peer < p && m.src + m.bytes <= slice * (size_t)p);
                CHECK(m.dst >= (size_t)r * cap && m.dst + m.bytes <= (size_t)(r + 1) * cap);
                memcpy(&stage[(size_t)m.peer][half + m.dst], &send[(size_t)r][m.src], m.bytes);
              }
            }
          // what a reduce_scatter consumer folds: slot [r] of rank d holds chunk c of slice d of rank r
          const size_t base = c * slot, len = clamp(slice, base, slot);
          for (int d = 0; d < p; ++d)
            for (int r = 0; r < p; ++r)
              CHECK(memcmp(&stage[(size_t)d][half + (size_t)r * cap], &send[(size_t)r][(size_t)d * slice + base], len) == 0);
          for (int r = 0; r < p; ++r)
            for (unsigned part = 0; part < n_con; ++part) {
              const Share sh = share_of(slice, slot, c, part, n_con, tile);
              for (size_t t = 0; t < fan_tiles(sh, p); ++t) {
                const Move m = gather_consume(sh, t, p, slice, cap, tile);
                memcpy(&recv[(size_t)r][m.dst], &stage[(size_t)r][half + m.src], m.bytes);
              }
            }
        }
        for (int r = 0; r < p; ++r)
          for (int q = 0; q < p; ++q)
            CHECK(memcmp(&recv[(size_t)r][(size_t)q * slice], &send[(size_t)q][(size_t)r * slice], slice) == 0);
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// "Last CTA posts" arrival counters of the device kernels, modelled on the host.
//
// A group of G CTAs runs R rounds; in each round a CTA does its share and then arrives; the CTA whose
// arrival completes the round's count posts the round's flag.  The schedules of the library only gate
// round k+2 on the post of round k (the gate goes through the peers), so a fast CTA can arrive for round
// k+1 before a slow sibling arrived for round k.  The kernels count arrivals in two counters chosen by
// the round's parity, each wrapping at G (kernels/common.cuh, arrive_and_post): every round must be posted
// exactly once, by its last arrival, whatever the interleaving.  A single wrapping counter is shown to
// fail under the same schedules, which is why the parity matters.
// ---------------------------------------------------------------------------------------------------
static void test_arrival_counters() {
  std::mt19937 rng(4711);
  int single_counter_failures = 0;
  for (int trial = 0; trial < 400; ++trial) {
    const int G = 2 + (int)(rng() % 7), R = 3 + (int)(rng() % 10);
    for (int mode = 0; mode < 2; ++mode) {  // 0: parity counters (the library), 1: one counter (the old scheme)
      std::vector<int> next((size_t)G, 0);          // round each CTA arrives for next
      std::vector<int> arrived((size_t)R, 0), posted((size_t)R, 0);
      unsigned ctr[2] = {0, 0};
      bool ok = true;
      int done = 0;
      while (done < G) {
        // pick a CTA that may proceed: round k needs the post of round k-2
        std::vector<int> ready;
        for (int c = 0; c < G; ++c)
          if (next[(size_t)c] < R && (next[(size_t)c] < 2 || posted[(size_t)next[(size_t)c] - 2])) ready.push_back(c);
        if (ready.empty()) { ok = false; break; }  // nobody can move: a round was never posted
        // skew: prefer the lowest-numbered CTAs most of the time so that some run ahead
        const int c = ready[(rng() % 4) ? 0 : rng() % ready.size()];
        const int k = next[(size_t)c]++;
        arrived[(size_t)k]++;
        unsigned& n = ctr[mode == 0 ? (k & 1) : 0];
        const bool last = n == (unsigned)G - 1;
        n = last ? 0 : n + 1;                       // atomicInc(ctr, G - 1)
        if (last) {
          if (arrived[(size_t)k] != G || posted[(size_t)k]) ok = false;  // posted early, or twice
          posted[(size_t)k] = 1;
        }
        if (next[(size_t)c] == R) ++done;
      }
      for (int k = 0; k < R; ++k) ok = ok && posted[(size_t)k] == 1;
      if (mode == 0) CHECK(ok);
      else if (!ok) ++single_counter_failures;
    }
  }
  CHECK(single_counter_failures > 0);  // the schedules really do exercise the hazard
}

// ---------------------------------------------------------------------------------------------------
// The ring-pipelined NVLS allreduce (kernels/nvls.cu): IN, RED and OUT groups of CTAs, chunks in a ring of D
// staging slots, the RED group split into two sub-groups that take the even and the odd chunks and post
// into a flag word per parity.  Model one rank (the ranks are symmetric): CTAs advance in random order,
// each group counts arrivals in the counter of ring slot c % D.  Checked: every chunk's A, B and C flag is
// posted exactly once and only after all CTAs of the responsible (sub-)group arrived for it; flag words
// only ever grow; a slot is never written by IN before OUT has emptied it.
// ---------------------------------------------------------------------------------------------------
static void test_ring_pipeline_schedule() {
  std::mt19937 rng(99);
  for (int trial = 0; trial < 300; ++trial) {
    const int D = 2 + (int)(rng() % 7);                  // 2..8 slots
    const int G = 1 + (int)(rng() % 20);                 // chunks
    const int n_in = 1 + (int)(rng() % 4), n_out = 1 + (int)(rng() % 4);
    const int n_red = 2 + (int)(rng() % 10);
    const int nsub = (n_red >= 8 && D >= 4) ? 2 : 1;
    struct Cta { int group, sub, next; };               // group 0 IN, 1 RED, 2 OUT; next = chunk it arrives for next
    std::vector<Cta> ctas;
    for (int i = 0; i < n_in; ++i) ctas.push_back({0, 0, 0});
    for (int i = 0; i < n_red; ++i) ctas.push_back({1, i % nsub, i % nsub});
    for (int i = 0; i < n_out; ++i) ctas.push_back({2, 0, 0});
    auto group_size = [&](const Cta& c) {
      if (c.group == 0) return n_in;
      if (c.group == 2) return n_out;
      return n_red / nsub + (c.sub < n_red % nsub ? 1 : 0);
    };
    std::vector<int> A((size_t)G, 0), B((size_t)G, 0), C((size_t)G, 0), arrivals((size_t)(3 * G), 0);
    unsigned ctr[3][8] = {};
    long wordB[2] = {0, 0}, wordA = 0, wordC = 0;
    bool ok = true;
    size_t finished = 0;
    for (const Cta& c : ctas) finished += c.next >= G;   // the odd sub-group has nothing to do when there is one chunk
    while (finished < ctas.size() && ok) {
      std::vector<size_t> ready;
      for (size_t i = 0; i < ctas.size(); ++i) {
        const Cta& c = ctas[i];
        if (c.next >= G) continue;
        bool can = true;
        if (c.group == 0) can = c.next < D || C[(size_t)(c.next - D)];   // slot emptied by OUT
        if (c.group == 1) can = A[(size_t)c.next] != 0;                   // chunk copied in
        if (c.group == 2) can = B[(size_t)c.next] != 0;                   // chunk reduced
        if (can) ready.push_back(i);
      }
      if (ready.empty()) { ok = false; break; }
      Cta& c = ctas[ready[(rng() % 3) ? 0 : rng() % ready.size()]];
      const int k = c.next;
      if (c.group == 0 && k >= D && !C[(size_t)(k - D)]) ok = false;       // would overwrite a slot still in use
      arrivals[(size_t)(c.group * G + k)]++;
      unsigned& n = ctr[c.group][k % D];
      const unsigned g = (unsigned)group_size(c);
      const bool last = n == g - 1;
      n = last ? 0 : n + 1;
      if (last) {
        if (arrivals[(size_t)(c.group * G + k)] != (int)g) ok = false;     // posted before everybody arrived
        std::vector<int>& flag = c.group == 0 ? A : (c.group == 1 ? B : C);
        if (flag[(size_t)k]) ok = false;                                    // posted twice
        flag[(size_t)k] = 1;
        long& word = c.group == 0 ? wordA : (c.group == 1 ? wordB[k & 1] : wordC);
        if (word >= k + 1) ok = false;                                      // a flag word must only grow
        word = k + 1;
      }
      c.next += c.group == 1 ? nsub : 1;
      if (c.next >= G) ++finished;
    }
    for (int k = 0; k < G; ++k) ok = ok && A[(size_t)k] && B[(size_t)k] && C[(size_t)k];
    CHECK(ok);
  }
}

static void test_progress_thread_placement() {
  using Al::internal::choose_pe_core;
  using Al::internal::parse_cpulist;
  CHECK((parse_cpulist("0-3,8,10-11\n") == std::vector<int>{0, 1, 2, 3, 8, 10, 11}));
  CHECK(parse_cpulist("").empty() && (parse_cpulist("5") == std::vector<int>{5}));
  std::vector<int> allowed;
  for (int c = 0; c < 64; ++c) allowed.push_back(c);
  // a GPU on the second socket (cores 32-63): its ranks poll from there, stepping down from the top
  const std::vector<int> near = parse_cpulist("32-63");
  CHECK(choose_pe_core(allowed, near, 0) == 63 && choose_pe_core(allowed, near, 3) == 60);
  // a GPU on the first socket never gets a core of the second one
  CHECK(choose_pe_core(allowed, parse_cpulist("0-31"), 1) == 30);
  // cores outside the affinity mask are not used; unknown locality falls back to the allowed cores
  CHECK(choose_pe_core({0, 1, 2, 3}, near, 0) == 3 && choose_pe_core({4, 5, 40, 41}, near, 1) == 40);
  CHECK(choose_pe_core(allowed, {}, 2) == 61 && choose_pe_core({7}, near, 0) == -1);
}

int main() {
  test_meta();
  test_progress_thread_placement();
  test_arrival_counters();
  test_ring_pipeline_schedule();
  test_spsc();
  test_mpsc();
  test_allocator();
  test_pool();
  test_progress_engine();
  test_progress_engine_concurrent_start();
  test_progress_engine_slot_reuse();
  test_reduce_and_halves();
  test_lifecycle_and_trace();
  test_bulk_tile_plans();
  if (g_fail) { fprintf(stderr, "%d check(s) failed\n", g_fail); return 1; }
  printf("all unit tests passed\n");
  return 0;
}
