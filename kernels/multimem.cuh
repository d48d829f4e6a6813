// multimem.* instructions (NVLink SHARP): loads that the NVSwitch reduces over every GPU bound to a
// multicast object, and stores that it replicates into all of them.  Shared by the NVLS allreduce
// and the window kernels.  16-byte vectors; bf16 / f16 sums accumulate in fp32 inside the switch.
#pragma once
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

enum class NvOp { add, min, max };

template <typename T, NvOp OP> struct MM;

template <> struct MM<float, NvOp::add> {
  static __device__ __forceinline__ uint4 ld(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
#define AL_MM_16(T, TOK, OP, OPTOK)                                                                       \
  template <> struct MM<T, NvOp::OP> {                                                                    \
    static __device__ __forceinline__ uint4 ld(const void* mc) {                                          \
      uint4 v;                                                                                            \
      asm volatile("multimem.ld_reduce.relaxed.sys.global." OPTOK ".v4." TOK " {%0,%1,%2,%3}, [%4];"      \
                   : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");                    \
      return v;                                                                                           \
    }                                                                                                     \
  };
AL_MM_16(__nv_bfloat16, "bf16x2", add, "add.acc::f32")
AL_MM_16(__nv_bfloat16, "bf16x2", min, "min")
AL_MM_16(__nv_bfloat16, "bf16x2", max, "max")
AL_MM_16(__half, "f16x2", add, "add.acc::f32")
AL_MM_16(__half, "f16x2", min, "min")
AL_MM_16(__half, "f16x2", max, "max")
#undef AL_MM_16

__device__ __forceinline__ void mm_st(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T>
__device__ __forceinline__ uint4 scale_pack(uint4 v, float s) {
  union { uint4 u; T e[16 / sizeof(T)]; } x;
  x.u = v;
#pragma unroll
  for (int k = 0; k < (int)(16 / sizeof(T)); ++k) x.e[k] = Elem<T>::down(Elem<T>::up(x.e[k]) * s);
  return x.u;
}

}  // namespace device
}  // namespace internal
}  // namespace Al
