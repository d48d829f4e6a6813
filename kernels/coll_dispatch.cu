// Run-time dispatch from datatype tags to the compiled collective kernels.
#include "al/device/kernels.hpp"
#include "coll_launch.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {
bool is_int(DType t) {
  switch (t) {
    case DType::i8: case DType::u8: case DType::i16: case DType::u16:
    case DType::i32: case DType::u32: case DType::i64: case DType::u64: return true;
    default: return false;
  }
}
bool is_small_float(DType t) { return t == DType::f32 || t == DType::f16 || t == DType::bf16; }
bool mixed_triple_ok(DType i, DType w, DType o) {
  if (!is_small_float(i) || !is_small_float(w) || !is_small_float(o)) return false;
  // (in, wire, out) triples compiled in coll_mixed.cu
  struct Tr { DType i, w, o; };
  static const Tr ok[] = {
      {DType::f32, DType::bf16, DType::f32}, {DType::f32, DType::f16, DType::f32},
      {DType::bf16, DType::bf16, DType::f32}, {DType::f16, DType::f16, DType::f32},
      {DType::f32, DType::f32, DType::bf16}, {DType::f32, DType::f32, DType::f16},
      {DType::f32, DType::bf16, DType::bf16}, {DType::f32, DType::f16, DType::f16},
      {DType::bf16, DType::f32, DType::f32}, {DType::f16, DType::f32, DType::f32}};
  for (const auto& t : ok)
    if (t.i == i && t.w == w && t.o == o) return true;
  return false;
}
}  // namespace

bool collective_supported(DType in, DType wire, DType out, ReductionOperator op) {
  if (in == wire && wire == out) {
    if (is_int(in)) return true;
    if (in == DType::f32 || in == DType::f64 || in == DType::f16 || in == DType::bf16)
      return op != ReductionOperator::bor && op != ReductionOperator::band && op != ReductionOperator::bxor;
    return false;
  }
  return (op == ReductionOperator::sum || op == ReductionOperator::avg) && mixed_triple_ok(in, wire, out);
}

void launch_collective(const CollParams& P, DType in, DType wire, DType out, int ctas, int threads,
                       int local_ranks, cudaStream_t stream) {
  LaunchCfg cfg;
  cfg.grid = dim3((unsigned)ctas, (unsigned)local_ranks, 1);
  cfg.threads = threads;
  cfg.cooperative = local_ranks > 1;
  cfg.stream = stream;
  const DevColl kind = (DevColl)P.kind;
  const bool reduces = kind == DevColl::allreduce || kind == DevColl::reduce || kind == DevColl::reduce_scatter;
  if (in == wire && wire == out) {
    if (!reduces && in == DType::u8) return launch_coll_bytes(P, cfg);
    switch (in) {
      case DType::f32: return launch_coll_f32(P, cfg);
      case DType::f64: return launch_coll_f64(P, cfg);
      case DType::f16: return launch_coll_f16(P, cfg);
      case DType::bf16: return launch_coll_bf16(P, cfg);
      default:
        if (is_int(in)) return launch_coll_int(P, in, cfg);
        throw_al_exception("datatype ", dtype_name(in), " is not supported on the device");
    }
  }
  if (!launch_coll_mixed(P, in, wire, out, cfg))
    throw_al_exception("no kernel for (in, wire, out) = (", dtype_name(in), ", ", dtype_name(wire), ", ",
                       dtype_name(out), ") with ", reduction_name((ReductionOperator)P.op));
}

}  // namespace device
}  // namespace internal
}  // namespace Al
