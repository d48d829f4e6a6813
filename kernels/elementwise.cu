// Stand-alone element-wise kernels: scale + dtype cast, fused momentum SGD over
// a flat parameter buffer, fill.  All are bandwidth bound; each thread moves
// 16 bytes per access and grids are sized in multiples of the SM count.
#include "al/cuda/cuda.hpp"
#include "al/device/kernels.hpp"
#include "datamove.cuh"

namespace Al {
namespace internal {
namespace device {

namespace {

constexpr int kThreads = 256;

int grid_for(size_t work_items) {
  // persistent-style grid: 148 SMs x 8 CTAs of 256 threads covers the machine
  size_t blocks = (work_items + kThreads - 1) / kThreads;
  const size_t cap = 148 * 8;
  if (blocks > cap) blocks = cap;
  if (blocks == 0) blocks = 1;
  return (int)blocks;
}

template <typename Ti, typename To>
__global__ void __launch_bounds__(kThreads) scale_cast_kernel(To* __restrict__ out, const Ti* __restrict__ in,
                                                               size_t n, float scale) {
  constexpr int VEC = 16 / (sizeof(Ti) > sizeof(To) ? sizeof(Ti) : sizeof(To));  // widest side moves 16 B
  using Ai = typename Elem<Ti>::Acc;
  using Ao = typename Elem<To>::Acc;
  const bool aligned = ((uintptr_t)in % (VEC * sizeof(Ti)) == 0) && ((uintptr_t)out % (VEC * sizeof(To)) == 0);
  const size_t nvec = aligned ? n / VEC : 0;
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  struct alignas(VEC * sizeof(Ti)) PI { Ti e[VEC]; };
  struct alignas(VEC * sizeof(To)) PO { To e[VEC]; };
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    PI a = ((const PI*)in)[v];
    PO o;
#pragma unroll
    for (int k = 0; k < VEC; ++k) o.e[k] = Elem<To>::down((Ao)((Ai)Elem<Ti>::up(a.e[k]) * (Ai)scale));
    ((PO*)out)[v] = o;
  }
  for (size_t i = nvec * VEC + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out[i] = Elem<To>::down((Ao)((Ai)Elem<Ti>::up(in[i]) * (Ai)scale));
}

template <typename Ti, typename To>
void run_scale_cast(void* out, const void* in, size_t n, double scale, cudaStream_t s) {
  if (n == 0) return;
  constexpr int VEC = 16 / (sizeof(Ti) > sizeof(To) ? sizeof(Ti) : sizeof(To));
  scale_cast_kernel<Ti, To><<<grid_for(n / VEC + 1), kThreads, 0, s>>>((To*)out, (const Ti*)in, n, (float)scale);
  AL_CHECK_CUDA(cudaGetLastError());
}

__global__ void __launch_bounds__(kThreads) scale_f64_kernel(double* out, const double* in, size_t n, double scale) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = in[i] * scale;
}

__global__ void __launch_bounds__(kThreads) sgd_momentum_kernel(float* __restrict__ param, float* __restrict__ mom,
                                                                 float* __restrict__ grad, size_t n, float lr,
                                                                 float mu, float wd, float gscale, int first,
                                                                 int zero_grad) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const bool aligned = (((uintptr_t)param | (uintptr_t)mom | (uintptr_t)grad) & 15) == 0;
  const size_t nvec = aligned ? n / 4 : 0;
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
    float4 p = ((float4*)param)[v];
    float4 g = ((float4*)grad)[v];
    float4 m = first ? make_float4(0.f, 0.f, 0.f, 0.f) : ((float4*)mom)[v];
    float* pp = (float*)&p; float* gg = (float*)&g; float* mm = (float*)&m;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float ge = gg[k] * gscale + wd * pp[k];
      mm[k] = first ? ge : mu * mm[k] + ge;
      pp[k] -= lr * mm[k];
    }
    ((float4*)param)[v] = p;
    ((float4*)mom)[v] = m;
    if (zero_grad) ((float4*)grad)[v] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (size_t i = nvec * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
    const float ge = grad[i] * gscale + wd * param[i];
    const float m = first ? ge : mu * mom[i] + ge;
    mom[i] = m;
    param[i] -= lr * m;
    if (zero_grad) grad[i] = 0.f;
  }
}

__global__ void __launch_bounds__(kThreads) fill_u32_kernel(uint32_t* out, size_t n, uint32_t value) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  const size_t nvec = (((uintptr_t)out & 15) == 0) ? n / 4 : 0;
  const uint4 v4 = make_uint4(value, value, value, value);
  for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) ((uint4*)out)[v] = v4;
  for (size_t i = nvec * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = value;
}

}  // namespace

void launch_scale_cast(void* out, DType out_dt, const void* in, DType in_dt, size_t n, double scale,
                       cudaStream_t stream) {
  using bf = __nv_bfloat16;
  using hf = __half;
#define AL_SC(DI, DO, TI, TO) \
  if (in_dt == DType::DI && out_dt == DType::DO) return run_scale_cast<TI, TO>(out, in, n, scale, stream);
  AL_SC(f32, f32, float, float)
  AL_SC(f32, bf16, float, bf)
  AL_SC(f32, f16, float, hf)
  AL_SC(bf16, f32, bf, float)
  AL_SC(f16, f32, hf, float)
  AL_SC(bf16, bf16, bf, bf)
  AL_SC(f16, f16, hf, hf)
  AL_SC(bf16, f16, bf, hf)
  AL_SC(f16, bf16, hf, bf)
#undef AL_SC
  if (in_dt == DType::f64 && out_dt == DType::f64) {
    if (n == 0) return;
    scale_f64_kernel<<<grid_for(n), kThreads, 0, stream>>>((double*)out, (const double*)in, n, scale);
    AL_CHECK_CUDA(cudaGetLastError());
    return;
  }
  throw_al_exception("scale_cast: unsupported type pair ", dtype_name(in_dt), " -> ", dtype_name(out_dt));
}

void launch_sgd_momentum(float* param, float* momentum, float* grad, size_t n, float lr, float mu,
                         float weight_decay, float grad_scale, int first_step, int zero_grad,
                         cudaStream_t stream) {
  if (n == 0) return;
  sgd_momentum_kernel<<<grid_for(n / 4 + 1), kThreads, 0, stream>>>(param, momentum, grad, n, lr, mu, weight_decay,
                                                                  grad_scale, first_step, zero_grad);
  AL_CHECK_CUDA(cudaGetLastError());
}

void launch_fill_u32(uint32_t* out, size_t n, uint32_t value, cudaStream_t stream) {
  if (n == 0) return;
  fill_u32_kernel<<<grid_for(n / 4 + 1), kThreads, 0, stream>>>(out, n, value);
  AL_CHECK_CUDA(cudaGetLastError());
}

}  // namespace device
}  // namespace internal
}  // namespace Al
