// Launch helpers shared by the per-type instantiation files of the collective kernel.
#pragma once
#include "al/cuda/cuda.hpp"
#include "coll_kernel.cuh"

namespace Al {
namespace internal {
namespace device {

struct LaunchCfg {
  dim3 grid;
  int threads;
  bool cooperative;
  cudaStream_t stream;
};

template <typename Ti, typename Tw, typename To, int FAM = kFamAll, typename Red>
void do_launch(const CollParams& P, Red red, const LaunchCfg& cfg) {
  if (!family_serves(FAM, (DevColl)P.kind))
    throw_al_exception("internal error: collective kernel family ", FAM, " launched for operation ", P.kind);
  void* args[] = {(void*)&P, (void*)&red};
  auto k = coll_kernel<Ti, Tw, To, Red, FAM>;
  if (cfg.cooperative)
    AL_CHECK_CUDA(cudaLaunchCooperativeKernel((const void*)k, cfg.grid, dim3((unsigned)cfg.threads), args, 0, cfg.stream));
  else
    AL_CHECK_CUDA(cudaLaunchKernel((const void*)k, cfg.grid, dim3((unsigned)cfg.threads), args, 0, cfg.stream));
}

/** Floating-point element types: dedicated kernels for sum / min / max, run-time operator otherwise.
 *  FAM = kFamReduce for one element type throughout (operations that only move data run as bytes). */
template <typename Ti, typename Tw, typename To, int FAM = kFamAll>
void launch_float(const CollParams& P, const LaunchCfg& cfg) {
  switch ((ReductionOperator)P.op) {
    case ReductionOperator::sum:
    case ReductionOperator::avg: do_launch<Ti, Tw, To, FAM>(P, RedSum(), cfg); break;
    case ReductionOperator::min: do_launch<Ti, Tw, To, FAM>(P, RedMin(), cfg); break;
    case ReductionOperator::max: do_launch<Ti, Tw, To, FAM>(P, RedMax(), cfg); break;
    default: do_launch<Ti, Tw, To, FAM>(P, RedRuntime{P.op}, cfg); break;
  }
}

/** Integer element types: one reducing kernel with the operator chosen at run time. */
template <typename T>
void launch_int(const CollParams& P, const LaunchCfg& cfg) {
  do_launch<T, T, T, kFamReduce>(P, RedRuntime{P.op}, cfg);
}

// Implemented one per file so that the instantiations compile in parallel.
void launch_coll_f32(const CollParams& P, const LaunchCfg& cfg);
void launch_coll_f64(const CollParams& P, const LaunchCfg& cfg);
void launch_coll_f16(const CollParams& P, const LaunchCfg& cfg);
void launch_coll_bf16(const CollParams& P, const LaunchCfg& cfg);
void launch_coll_int(const CollParams& P, DType dt, const LaunchCfg& cfg);
void launch_coll_bytes(const CollParams& P, const LaunchCfg& cfg);
/** Mixed-type sum: (in, wire, out) among f32 / f16 / bf16. Returns false when the triple is not compiled. */
bool launch_coll_mixed(const CollParams& P, DType ti, DType tw, DType to, const LaunchCfg& cfg);

}  // namespace device
}  // namespace internal
}  // namespace Al
