// Collective kernel instantiations for __nv_bfloat16 elements.
#include "coll_launch.cuh"
namespace Al { namespace internal { namespace device {
void launch_coll_bf16(const CollParams& P, const LaunchCfg& cfg) { launch_float<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, kFamReduce>(P, cfg); }
}}}
