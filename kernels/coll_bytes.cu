// Collective kernel instantiation for pure data movement (counts in bytes).
#include "coll_launch.cuh"
namespace Al { namespace internal { namespace device {
void launch_coll_bytes(const CollParams& P, const LaunchCfg& cfg) {
  do_launch<unsigned char, unsigned char, unsigned char, kFamMove>(P, RedNone(), cfg);
}
}}}
