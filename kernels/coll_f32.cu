// Collective kernel instantiations for float elements.
#include "coll_launch.cuh"
namespace Al { namespace internal { namespace device {
void launch_coll_f32(const CollParams& P, const LaunchCfg& cfg) { launch_float<float, float, float, kFamReduce>(P, cfg); }
}}}
