/**
 * @file tuning.hpp
 * Run-time tuning table: progress-engine limits, pool sizes, staging sizes,
 * algorithm cross-over points and CTA budgets of the device kernels.
 *
 * The reference fixes these at configure time (CMakeLists.txt:166-215 ->
 * cmake/tuning_params.hpp.in:36-89).  Here every value has an environment
 * variable of the same spirit (AL_<NAME>) read once at Initialize(), and can
 * be changed programmatically through Al::tuning() before communicators are
 * created.
 */
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>

#include "al/config.hpp"

namespace Al {

/**
 * Message sizes at which the device backend changes algorithm.  They depend on the number of ranks, so
 * the table has a row for communicators of 2, of 3-4 and of 5-8 ranks (tuned on 2, 4 and 8 B200 over
 * NVLink 5 / NVSwitch; al_info prints it).  Every entry has an environment variable that sets all rows
 * (AL_LL_MAX, ...) and one per row (AL_LL_MAX_P2, _P4, _P8); al_set_tuning("ll_max_bytes", v) sets all
 * rows, "ll_max_bytes@4" one.
 */
struct Crossovers {
  size_t ll_max_bytes;             ///< AL_LL_MAX: at most this many bytes per pair of ranks travel as low-latency packets (hard limit 1 MiB; 0 = never)
  size_t ar_oneshot_max_bytes;     ///< AL_AR_ONESHOT_MAX: staged one-shot allreduce up to this size
  size_t ar_nvls_min_bytes;        ///< AL_AR_NVLS_MIN: NVLS allreduce from this size on
  size_t ar_pipeline_min_bytes;    ///< AL_AR_PIPELINE_MIN: two ranks: the one-shot allreduce splits its grid into pushing and reducing CTAs from this size on
  size_t nvls_pipeline_min_bytes;  ///< AL_NVLS_PIPELINE_MIN: staged NVLS allreduce is software-pipelined from this size on
  size_t pipeline_min_bytes;       ///< AL_PIPELINE_MIN: per-rank slice from which staged reduce_scatter / allgather / alltoall split the grid into publishers and consumers
  size_t window_min_bytes;         ///< AL_WINDOW_MIN: total message size from which registered buffers take the window kernels (below: staging or packets, one flag round less)
  size_t ar_ll_max_bytes;          ///< AL_AR_LL_MAX: allreduce travels as one-phase packets (every rank sends its whole vector to every rank) up to this size; at most ll_max_bytes
  size_t ar_ll2_max_bytes;         ///< AL_AR_LL2_MAX: allreduce up to this size (beyond ll_max_bytes) runs as packets in two phases (reduce-scatter, then allgather; more than two ranks; hard limit p x 512 KiB)
  size_t rs_nvls_min_bytes;        ///< AL_RS_NVLS_MIN: total message size from which reduce_scatter of private buffers reduces in the switch (staged NVLS; needs multicast and more than two ranks)
};

struct Tuning {
  // ---- progress engine ------------------------------------------------------
  int pe_num_concurrent_ops = AL_PE_NUM_CONCURRENT_OPS_DEFAULT;  ///< AL_PE_NUM_CONCURRENT_OPS
  bool pe_start_on_demand = true;                                ///< AL_PE_START_ON_DEMAND
  bool pe_bind_thread = true;                                    ///< AL_PE_BIND (pin the PE thread to a core)
  double pe_hang_seconds = 10.0;                                 ///< AL_PE_HANG_SECONDS (watchdog threshold, <=0 off)
  // ---- pools ----------------------------------------------------------------
  int sync_mem_prealloc = AL_SYNC_MEM_PREALLOC_DEFAULT;          ///< AL_SYNC_MEM_PREALLOC
  int stream_pool_size = AL_CUDA_STREAM_POOL_SIZE_DEFAULT;       ///< AL_CUDA_STREAM_POOL_SIZE
  bool disable_background_streams = false;                       ///< AL_DISABLE_BACKGROUND_STREAMS
  // ---- host (shared-memory) backend -----------------------------------------
  size_t host_stage_bytes = size_t{4} << 20;   ///< AL_HOST_STAGE_BYTES: one staging half per rank
  size_t host_mailbox_bytes = size_t{128} << 10;  ///< AL_HOST_MAILBOX_BYTES: one p2p slot per ordered pair
  double host_wait_timeout_s = 120.0;          ///< AL_HOST_WAIT_TIMEOUT_S: a peer that never arrives raises
  bool host_two_level = true;                  ///< AL_HOST_TWO_LEVEL: across nodes, small allreduce / bcast and every barrier go through shared memory inside each node and sockets between the nodes' first ranks
  size_t host_two_level_max_bytes = size_t{32} << 10;  ///< AL_HOST_TWO_LEVEL_MAX: largest message that takes the two-level path (larger ones use every rank's connections)
  bool host_serialize = false;                 ///< AL_HOST_SERIALIZE: blocking host calls also run on the progress thread (the reference's ALUMINUM_MPI_SERIALIZE)
  // ---- device backend ---------------------------------------------------------
  size_t dev_stage_bytes = size_t{64} << 20;   ///< AL_DEV_STAGE_BYTES: one staging half per rank per communicator
  size_t dev_mailbox_bytes = size_t{8} << 20;  ///< AL_DEV_MAILBOX_BYTES: size of one p2p mailbox slot (larger pieces amortise the per-piece flag round: 4 MiB moved 315 GB/s, 16 MiB 536 GB/s between two B200)
  int dev_mailbox_slots = 2;                   ///< AL_DEV_MAILBOX_SLOTS: slots of the ring every ordered pair of ranks owns (pieces in flight per transfer)
  size_t p2p_ll_max_bytes = size_t{2} << 20;       ///< AL_P2P_LL_MAX: point-to-point messages up to this size travel as low-latency packets (data and piece number in one 16-byte store).  A communicator sizes its packet slots (ranks x ring depth x twice this) when it is created; lowering the value later takes effect at once, raising it applies to new communicators.  At most 8 MiB; 0 = never
  size_t p2p_rendezvous_bytes = size_t{1} << 20;  ///< AL_P2P_RENDEZVOUS: from this size on a send first waits for the receiver and, if the receive buffer is registered, stores straight into it (0 = never)
  double dev_wait_timeout_ms = 20000.0;        ///< AL_DEV_WAIT_TIMEOUT_MS: bound of every device-side flag wait
  bool dev_enable_nvls = true;                 ///< AL_DEV_NVLS: bind staging to an NVLink multicast object when supported
  int max_ctas = 128;                          ///< AL_MAX_CTAS_PER_OP: CTA budget of a bandwidth kernel
  int max_ctas_pipelined = 128;                ///< AL_MAX_CTAS_PIPELINED: grid of the pipelined reduce_scatter / allgather / alltoall (half publishes, half consumes; at most one CTA per SM)
  int max_ctas_nvls = 128;                     ///< AL_MAX_CTAS_NVLS: staged NVLS allreduce (its copies need many CTAs)
  size_t nvls_chunk_bytes = size_t{16} << 20;  ///< AL_NVLS_CHUNK_BYTES: smallest chunk of the pipelined staged NVLS allreduce (a chunk is 1/16 of the message, at least this, at most a staging half)
  int max_ctas_zero_copy = 32;                 ///< AL_MAX_CTAS_ZERO_COPY: NVLS allreduce on symmetric buffers (no copies)
  int threads_per_cta = 512;                   ///< AL_THREADS_PER_CTA
  int p2p_max_ctas = 64;                       ///< AL_DEV_P2P_CTAS: most CTAs one send or receive of a point-to-point launch gets (one per 64 KiB of a mailbox piece)
  bool bulk_pipeline = false;                  ///< AL_DEV_BULK_PIPELINE: pipelined reduce_scatter / allgather / alltoall move their data with the bulk copy engine (cp.async.bulk) when every buffer is 16-byte aligned
  int bulk_pub_ctas = 16;                      ///< AL_DEV_BULK_PUB_CTAS: publishing CTAs of that kernel (one issuing thread each)
  int bulk_con_ctas = 16;                      ///< AL_DEV_BULK_CON_CTAS: its consuming CTAs for allgather / alltoall (reduce_scatter reduces with SM loads and takes max_ctas/2)
  int ll_max_ctas = 64;                        ///< AL_LL_CTAS: most CTAs of a low-latency launch (256 threads, one 16-byte group each)
  Crossovers cross[3] = {
      // ll_max      one-shot max      nvls min  ar pipeline   nvls pipeline      rs/ag/a2a pipeline  window min  one-phase / two-phase packet allreduce max  rs nvls min
      {size_t{1} << 20, size_t{2} << 20, 0, size_t{64} << 20, size_t{128} << 20, size_t{32} << 20, size_t{16} << 20, size_t{1} << 20, 0, ~size_t{0}},                       // 2 ranks
      {size_t{256} << 10, size_t{256} << 10, 0, size_t{64} << 20, size_t{64} << 20, size_t{32} << 20, size_t{16} << 20, size_t{256} << 10, size_t{2} << 20, ~size_t{0}},   // 3-4 ranks
      {size_t{256} << 10, size_t{16} << 10, 0, size_t{64} << 20, size_t{64} << 20, size_t{32} << 20, size_t{16} << 20, size_t{64} << 10, size_t{2} << 20, ~size_t{0}},     // 5-8 ranks
  };
  /** Row of the table for a communicator of `p` ranks. */
  const Crossovers& crossovers(int p) const { return cross[p <= 2 ? 0 : (p <= 4 ? 1 : 2)]; }
  bool window_enable = true;                   ///< AL_WINDOW: uniform reduce_scatter / allgather / alltoall / bcast on registered (or symm_alloc) buffers skip the staging area
  int window_ctas = 128;                       ///< AL_WINDOW_CTAS: CTA budget of a window kernel
  int window_multimem_ag_ranks = 16;          ///< AL_WINDOW_MULTIMEM_AG_RANKS: allgather uses multimem.st from this many ranks on (a multicast store returns to its sender too, which costs 1/(p-1) extra ingress)
  int window_rs_min_ranks = 5;                 ///< AL_WINDOW_RS_MIN_RANKS: automatic reduce_scatter takes the window path (switch reduction) from this many ranks on (4 ranks: the staged push measured 5-8 % faster)
  size_t window_rs_min_bytes = size_t{32} << 20;  ///< AL_WINDOW_RS_MIN: ... and from this total size on (8 ranks: 16 MiB 51 us on the window path against 47 us staged, 64 MiB 121 against 128)
  bool window_multimem = true;                 ///< AL_WINDOW_MULTIMEM: let window kernels use multimem.st / multimem.ld_reduce when all ranks pass the same offset of one multicast-bound window
  // ---- diagnostics ------------------------------------------------------------
  bool trace = false;                          ///< AL_TRACE: record every API call
  bool debug_checks = false;                   ///< AL_DEBUG: argument checks on every call
  bool debug_guard = false;                    ///< AL_DEBUG_GUARD: guard regions around every symm_alloc block, verified by check_guards() and symm_free()
  bool signal_handler = true;                  ///< !AL_DISABLE_SIGNAL_HANDLER

  // ---- host-side fault injection (tests only; nothing here touches a GPU) -------
  int fault_rank = -1;                         ///< AL_FAULT_RANK: world rank that misbehaves (-1: nobody)
  long fault_op = 0;                           ///< AL_FAULT_OP: which host collective of a communicator (1 = its first)
  int fault_kind = 0;                          ///< AL_FAULT_KIND: 0 none, 1 the rank never signals that op, 2 it signals AL_FAULT_DELAY_MS late
  long fault_delay_ms = 0;                     ///< AL_FAULT_DELAY_MS
  long fault_jitter_us = 0;                    ///< AL_FAULT_JITTER_US: every rank sleeps a random time below this before each publish

  /** Re-read every AL_* environment variable. */
  void load_from_env();
  /** One "name = value" line per entry, for al_info. */
  std::string describe() const;
};

/** The process-wide table. */
Tuning& tuning();

}  // namespace Al
