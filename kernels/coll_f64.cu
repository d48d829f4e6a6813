// Collective kernel instantiations for double elements.
#include "coll_launch.cuh"
namespace Al { namespace internal { namespace device {
void launch_coll_f64(const CollParams& P, const LaunchCfg& cfg) { launch_float<double, double, double, kFamReduce>(P, cfg); }
}}}
