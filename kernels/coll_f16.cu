// Collective kernel instantiations for __half elements.
#include "coll_launch.cuh"
namespace Al { namespace internal { namespace device {
void launch_coll_f16(const CollParams& P, const LaunchCfg& cfg) { launch_float<__half, __half, __half, kFamReduce>(P, cfg); }
}}}
