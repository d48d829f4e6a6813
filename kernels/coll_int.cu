// Collective kernel instantiations for integer elements (operator chosen at run time).
#include "coll_launch.cuh"
namespace Al { namespace internal { namespace device {
void launch_coll_int(const CollParams& P, DType dt, const LaunchCfg& cfg) {
  switch (dt) {
    case DType::i8: launch_int<signed char>(P, cfg); break;
    case DType::u8: launch_int<unsigned char>(P, cfg); break;
    case DType::i16: launch_int<short>(P, cfg); break;
    case DType::u16: launch_int<unsigned short>(P, cfg); break;
    case DType::i32: launch_int<int>(P, cfg); break;
    case DType::u32: launch_int<unsigned int>(P, cfg); break;
    case DType::i64: launch_int<long long>(P, cfg); break;
    case DType::u64: launch_int<unsigned long long>(P, cfg); break;
    default: throw_al_exception("not an integer datatype: ", dtype_name(dt));
  }
}
}}}
