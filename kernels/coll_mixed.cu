// Collective kernel instantiations whose input, wire and output types differ:
// the dtype cast is fused into the publish step (input -> wire) and into the
// final store (accumulator -> output), so no separate cast kernel runs.
#include "coll_launch.cuh"
namespace Al { namespace internal { namespace device {
bool launch_coll_mixed(const CollParams& P, DType ti, DType tw, DType to, const LaunchCfg& cfg) {
  using bf = __nv_bfloat16;
  using hf = __half;
#define AL_MIX(TI, TW, TO, CI, CW, CO)                                              \
  if (ti == DType::TI && tw == DType::TW && to == DType::TO) {                      \
    do_launch<CI, CW, CO>(P, RedSum(), cfg);                                        \
    return true;                                                                    \
  }
  const ReductionOperator op = (ReductionOperator)P.op;
  if (op != ReductionOperator::sum && op != ReductionOperator::avg) return false;
  AL_MIX(f32, bf16, f32, float, bf, float)    // compressed wire
  AL_MIX(f32, f16, f32, float, hf, float)
  AL_MIX(bf16, bf16, f32, bf, bf, float)      // low-precision in, fp32 out
  AL_MIX(f16, f16, f32, hf, hf, float)
  AL_MIX(f32, f32, bf16, float, float, bf)    // fp32 in, low-precision out
  AL_MIX(f32, f32, f16, float, float, hf)
  AL_MIX(f32, bf16, bf16, float, bf, bf)      // cast on publish (allgather with cast)
  AL_MIX(f32, f16, f16, float, hf, hf)
  AL_MIX(bf16, f32, f32, bf, float, float)
  AL_MIX(f16, f32, f32, hf, float, float)
#undef AL_MIX
  return false;
}
}}}
