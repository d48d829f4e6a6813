// Run-time tuning table (see al/tuning.hpp).
#include "al/tuning.hpp"

#include <algorithm>
#include <sstream>

#include "al/util/utils.hpp"

namespace Al {

Tuning& tuning() {
  static Tuning t = [] { Tuning x; x.load_from_env(); return x; }();
  return t;
}

void Tuning::load_from_env() {
  using internal::env_double;
  using internal::env_long;
  pe_num_concurrent_ops = (int)env_long("AL_PE_NUM_CONCURRENT_OPS", pe_num_concurrent_ops);
  pe_start_on_demand = env_long("AL_PE_START_ON_DEMAND", pe_start_on_demand) != 0;
  pe_bind_thread = env_long("AL_PE_BIND", pe_bind_thread) != 0;
  pe_hang_seconds = env_double("AL_PE_HANG_SECONDS", pe_hang_seconds);
  sync_mem_prealloc = (int)env_long("AL_SYNC_MEM_PREALLOC", sync_mem_prealloc);
  stream_pool_size = (int)env_long("AL_CUDA_STREAM_POOL_SIZE", stream_pool_size);
  disable_background_streams = env_long("AL_DISABLE_BACKGROUND_STREAMS", disable_background_streams) != 0;
  host_stage_bytes = (size_t)env_long("AL_HOST_STAGE_BYTES", (long)host_stage_bytes);
  host_mailbox_bytes = (size_t)env_long("AL_HOST_MAILBOX_BYTES", (long)host_mailbox_bytes);
  host_wait_timeout_s = env_double("AL_HOST_WAIT_TIMEOUT_S", host_wait_timeout_s);
  host_two_level = env_long("AL_HOST_TWO_LEVEL", host_two_level) != 0;
  host_two_level_max_bytes = (size_t)env_long("AL_HOST_TWO_LEVEL_MAX", (long)host_two_level_max_bytes);
  host_serialize = env_long("AL_HOST_SERIALIZE", host_serialize) != 0;
  dev_stage_bytes = (size_t)env_long("AL_DEV_STAGE_BYTES", (long)dev_stage_bytes);
  dev_mailbox_bytes = (size_t)env_long("AL_DEV_MAILBOX_BYTES", (long)dev_mailbox_bytes);
  dev_wait_timeout_ms = env_double("AL_DEV_WAIT_TIMEOUT_MS", dev_wait_timeout_ms);
  dev_enable_nvls = env_long("AL_DEV_NVLS", dev_enable_nvls) != 0;
  max_ctas = (int)env_long("AL_MAX_CTAS_PER_OP", max_ctas);
  max_ctas_nvls = (int)env_long("AL_MAX_CTAS_NVLS", max_ctas_nvls);
  max_ctas_zero_copy = (int)env_long("AL_MAX_CTAS_ZERO_COPY", max_ctas_zero_copy);
  threads_per_cta = (int)env_long("AL_THREADS_PER_CTA", threads_per_cta);
  p2p_max_ctas = (int)env_long("AL_DEV_P2P_CTAS", p2p_max_ctas);
  bulk_pipeline = env_long("AL_DEV_BULK_PIPELINE", bulk_pipeline) != 0;
  bulk_pub_ctas = (int)env_long("AL_DEV_BULK_PUB_CTAS", bulk_pub_ctas);
  bulk_con_ctas = (int)env_long("AL_DEV_BULK_CON_CTAS", bulk_con_ctas);
  ll_max_ctas = (int)env_long("AL_LL_CTAS", ll_max_ctas);
  max_ctas_pipelined = (int)env_long("AL_MAX_CTAS_PIPELINED", max_ctas_pipelined);
  nvls_chunk_bytes = (size_t)env_long("AL_NVLS_CHUNK_BYTES", (long)nvls_chunk_bytes);
  dev_mailbox_slots = (int)env_long("AL_DEV_MAILBOX_SLOTS", dev_mailbox_slots);
  p2p_rendezvous_bytes = (size_t)env_long("AL_P2P_RENDEZVOUS", (long)p2p_rendezvous_bytes);
  p2p_ll_max_bytes = (size_t)env_long("AL_P2P_LL_MAX", (long)p2p_ll_max_bytes);
  {
    struct Entry { const char* env; size_t Crossovers::*field; };
    static const Entry entries[] = {
        {"AL_LL_MAX", &Crossovers::ll_max_bytes}, {"AL_AR_ONESHOT_MAX", &Crossovers::ar_oneshot_max_bytes},
        {"AL_AR_NVLS_MIN", &Crossovers::ar_nvls_min_bytes}, {"AL_AR_PIPELINE_MIN", &Crossovers::ar_pipeline_min_bytes},
        {"AL_NVLS_PIPELINE_MIN", &Crossovers::nvls_pipeline_min_bytes}, {"AL_PIPELINE_MIN", &Crossovers::pipeline_min_bytes},
        {"AL_WINDOW_MIN", &Crossovers::window_min_bytes}, {"AL_RS_NVLS_MIN", &Crossovers::rs_nvls_min_bytes},
        {"AL_AR_LL2_MAX", &Crossovers::ar_ll2_max_bytes}, {"AL_AR_LL_MAX", &Crossovers::ar_ll_max_bytes}};
    static const char* suffix[3] = {"_P2", "_P4", "_P8"};
    for (const Entry& e : entries)
      for (int row = 0; row < 3; ++row) {
        long v = env_long(e.env, -1);
        v = env_long((std::string(e.env) + suffix[row]).c_str(), v);
        if (v >= 0) cross[row].*(e.field) = (size_t)v;
      }
  }
  window_enable = env_long("AL_WINDOW", window_enable) != 0;
  window_ctas = (int)env_long("AL_WINDOW_CTAS", window_ctas);
  window_multimem = env_long("AL_WINDOW_MULTIMEM", window_multimem) != 0;
  window_multimem_ag_ranks = (int)env_long("AL_WINDOW_MULTIMEM_AG_RANKS", window_multimem_ag_ranks);
  window_rs_min_ranks = (int)env_long("AL_WINDOW_RS_MIN_RANKS", window_rs_min_ranks);
  window_rs_min_bytes = (size_t)env_long("AL_WINDOW_RS_MIN", (long)window_rs_min_bytes);
  trace = env_long("AL_TRACE", trace) != 0;
#ifdef AL_DEBUG_DEFAULT
  debug_checks = true;   // built with ALUMINUM_ENABLE_DEBUG: checks are on unless AL_DEBUG=0
#endif
#ifdef AL_TRACE_DEFAULT
  trace = true;          // built with ALUMINUM_ENABLE_TRACE
#endif
  debug_checks = env_long("AL_DEBUG", debug_checks) != 0;
  debug_guard = env_long("AL_DEBUG_GUARD", debug_guard) != 0;
  signal_handler = env_long("AL_DISABLE_SIGNAL_HANDLER", 0) == 0;
  fault_rank = (int)env_long("AL_FAULT_RANK", fault_rank);
  fault_op = env_long("AL_FAULT_OP", fault_op);
  fault_kind = (int)env_long("AL_FAULT_KIND", fault_kind);
  fault_delay_ms = env_long("AL_FAULT_DELAY_MS", fault_delay_ms);
  fault_jitter_us = env_long("AL_FAULT_JITTER_US", fault_jitter_us);
  if (max_ctas < 1) max_ctas = 1;
  if (max_ctas > AL_MAX_CTAS) max_ctas = AL_MAX_CTAS;
  if (max_ctas_nvls < 1) max_ctas_nvls = 1;
  if (max_ctas_nvls > AL_MAX_CTAS) max_ctas_nvls = AL_MAX_CTAS;
  if (max_ctas_zero_copy < 1) max_ctas_zero_copy = 1;
  if (max_ctas_zero_copy > AL_MAX_CTAS) max_ctas_zero_copy = AL_MAX_CTAS;
  p2p_max_ctas = std::max(1, std::min(p2p_max_ctas, AL_MAX_CTAS / 2));
  bulk_pub_ctas = std::max(1, std::min(bulk_pub_ctas, AL_MAX_CTAS / 2));
  bulk_con_ctas = std::max(1, std::min(bulk_con_ctas, AL_MAX_CTAS / 2));
  if (threads_per_cta < 64) threads_per_cta = 64;
  if (threads_per_cta > 1024) threads_per_cta = 1024;
  threads_per_cta = threads_per_cta / 32 * 32;
  // staging halves must stay 16-byte divisible for every rank count up to 8
  dev_stage_bytes = dev_stage_bytes / 4096 * 4096;
  if (dev_stage_bytes < 65536) dev_stage_bytes = 65536;
  host_stage_bytes = host_stage_bytes / 4096 * 4096;
  if (host_stage_bytes < 4096) host_stage_bytes = 4096;
  if (host_mailbox_bytes < 256) host_mailbox_bytes = 256;
}

std::string Tuning::describe() const {
  std::ostringstream ss;
  ss << "pe_num_concurrent_ops = " << pe_num_concurrent_ops << "\n"
     << "pe_start_on_demand = " << pe_start_on_demand << "\n"
     << "pe_bind_thread = " << pe_bind_thread << "\n"
     << "pe_hang_seconds = " << pe_hang_seconds << "\n"
     << "pe_num_streams = " << AL_PE_NUM_STREAMS << "\n"
     << "pe_num_pipeline_stages = " << AL_PE_NUM_PIPELINE_STAGES << "\n"
     << "pe_input_queue_size = " << AL_PE_INPUT_QUEUE_SIZE << "\n"
     << "sync_mem_prealloc = " << sync_mem_prealloc << "\n"
     << "stream_pool_size = " << stream_pool_size << "\n"
     << "disable_background_streams = " << disable_background_streams << "\n"
     << "host_stage_bytes = " << host_stage_bytes << "\n"
     << "host_mailbox_bytes = " << host_mailbox_bytes << "\n"
     << "host_wait_timeout_s = " << host_wait_timeout_s << "\n"
     << "host_two_level = " << host_two_level << "\n"
     << "host_two_level_max_bytes = " << host_two_level_max_bytes << "\n"
     << "host_serialize = " << host_serialize << "\n"
     << "dev_stage_bytes = " << dev_stage_bytes << "\n"
     << "dev_mailbox_bytes = " << dev_mailbox_bytes << "\n"
     << "dev_wait_timeout_ms = " << dev_wait_timeout_ms << "\n"
     << "dev_enable_nvls = " << dev_enable_nvls << "\n"
     << "max_ctas = " << max_ctas << "\n"
     << "max_ctas_nvls = " << max_ctas_nvls << "\n"
     << "max_ctas_zero_copy = " << max_ctas_zero_copy << "\n"
     << "threads_per_cta = " << threads_per_cta << "\n"
     << "p2p_max_ctas = " << p2p_max_ctas << "\n"
     << "bulk_pipeline = " << bulk_pipeline << "\n"
     << "bulk_pub_ctas = " << bulk_pub_ctas << "\n"
     << "bulk_con_ctas = " << bulk_con_ctas << "\n"
     << "ll_max_ctas = " << ll_max_ctas << "\n"
     << "max_ctas_pipelined = " << max_ctas_pipelined << "\n"
     << "nvls_chunk_bytes = " << nvls_chunk_bytes << "\n"
     << "dev_mailbox_slots = " << dev_mailbox_slots << "\n"
     << "p2p_rendezvous_bytes = " << p2p_rendezvous_bytes << "\n"
     << "p2p_ll_max_bytes = " << p2p_ll_max_bytes << "\n"
     << "window_enable = " << window_enable << "\n"
     << "window_ctas = " << window_ctas << "\n"
     << "window_multimem = " << window_multimem << "\n"
     << "window_multimem_ag_ranks = " << window_multimem_ag_ranks << "\n"
     << "window_rs_min_ranks = " << window_rs_min_ranks << "\n"
     << "window_rs_min_bytes = " << window_rs_min_bytes << "\n"
     << "crossovers (bytes)      2 ranks      3-4 ranks      5-8 ranks\n"
     << "  ll_max_bytes            " << cross[0].ll_max_bytes << "  " << cross[1].ll_max_bytes << "  " << cross[2].ll_max_bytes << "\n"
     << "  ar_oneshot_max_bytes    " << cross[0].ar_oneshot_max_bytes << "  " << cross[1].ar_oneshot_max_bytes << "  " << cross[2].ar_oneshot_max_bytes << "\n"
     << "  ar_nvls_min_bytes       " << cross[0].ar_nvls_min_bytes << "  " << cross[1].ar_nvls_min_bytes << "  " << cross[2].ar_nvls_min_bytes << "\n"
     << "  ar_pipeline_min_bytes   " << cross[0].ar_pipeline_min_bytes << "  " << cross[1].ar_pipeline_min_bytes << "  " << cross[2].ar_pipeline_min_bytes << "\n"
     << "  nvls_pipeline_min_bytes " << cross[0].nvls_pipeline_min_bytes << "  " << cross[1].nvls_pipeline_min_bytes << "  " << cross[2].nvls_pipeline_min_bytes << "\n"
     << "  pipeline_min_bytes      " << cross[0].pipeline_min_bytes << "  " << cross[1].pipeline_min_bytes << "  " << cross[2].pipeline_min_bytes << "\n"
     << "  window_min_bytes        " << cross[0].window_min_bytes << "  " << cross[1].window_min_bytes << "  " << cross[2].window_min_bytes << "\n"
     << "  ar_ll_max_bytes         " << cross[0].ar_ll_max_bytes << "  " << cross[1].ar_ll_max_bytes << "  " << cross[2].ar_ll_max_bytes << "\n"
     << "  ar_ll2_max_bytes        " << cross[0].ar_ll2_max_bytes << "  " << cross[1].ar_ll2_max_bytes << "  " << cross[2].ar_ll2_max_bytes << "\n"
     << "  rs_nvls_min_bytes       " << cross[0].rs_nvls_min_bytes << "  " << cross[1].rs_nvls_min_bytes << "  " << cross[2].rs_nvls_min_bytes << "\n"
     << "trace = " << trace << "\n"
     << "debug_checks = " << debug_checks << "\n"
     << "debug_guard = " << debug_guard << "\n"
     << "signal_handler = " << signal_handler << "\n"
     << "fault_rank = " << fault_rank << "\n"
     << "fault_op = " << fault_op << "\n"
     << "fault_kind = " << fault_kind << "\n"
     << "fault_delay_ms = " << fault_delay_ms << "\n"
     << "fault_jitter_us = " << fault_jitter_us << "\n";
  return ss.str();
}

}  // namespace Al
