/**
 * @file cuda.hpp
 * CUDA layer basics: error-check macros, lazily resolved driver entry points,
 * init/finalize of the stream pool and the pinned flag pool.
 *
 * Parity: include/aluminum/cuda/cuda.hpp:55-126 (AL_CHECK_CUDA*,
 * AL_FORCE_CHECK_GPU*), src/cuda/cuda.cpp:44-88 (cuda::init / finalize,
 * stream_memory_operations_supported).  The driver API is never linked: the
 * few driver functions used (stream write/wait value, virtual memory and
 * multicast management) are looked up through cudaGetDriverEntryPoint on
 * first use, so the library loads on hosts that have no driver installed.
 */
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include "al/base.hpp"

#define AL_CHECK_CUDA(call)                                                              \
  do {                                                                                   \
    cudaError_t al_e_ = (call);                                                          \
    if (al_e_ != cudaSuccess) {                                                          \
      throw_al_exception("CUDA error: ", cudaGetErrorName(al_e_), " (",                 \
                         cudaGetErrorString(al_e_), ") in " #call);                      \
    }                                                                                    \
  } while (0)
#define AL_CHECK_CUDA_NOSYNC(call) AL_CHECK_CUDA(call)
#define AL_FORCE_CHECK_GPU(call) AL_CHECK_CUDA(call)
#define AL_FORCE_CHECK_GPU_NOSYNC(call) AL_CHECK_CUDA(call)
#define AL_GPU_SYNC() AL_CHECK_CUDA(cudaDeviceSynchronize())
/** For destructors and other contexts that must not throw. */
#define AL_WARN_CUDA(call)                                                               \
  do {                                                                                   \
    cudaError_t al_e_ = (call);                                                          \
    if (al_e_ != cudaSuccess && al_e_ != cudaErrorCudartUnloading) {                     \
      std::cerr << "[al] CUDA warning: " << cudaGetErrorName(al_e_) << " in " #call "\n"; \
      (void)cudaGetLastError();                                                          \
    }                                                                                    \
  } while (0)
#define AL_CHECK_CUDA_DRV(call)                                                          \
  do {                                                                                   \
    CUresult al_r_ = (call);                                                             \
    if (al_r_ != CUDA_SUCCESS) {                                                         \
      throw_al_exception("CUDA driver error ", ::Al::internal::cuda::drv_error_name(al_r_), \
                         " in " #call);                                                  \
    }                                                                                    \
  } while (0)
#define AL_FORCE_CHECK_GPU_DRV(call) AL_CHECK_CUDA_DRV(call)
#define AL_FORCE_CHECK_GPU_DRV_NOSYNC(call) AL_CHECK_CUDA_DRV(call)

namespace Al {
namespace internal {
namespace cuda {

/** Driver entry points resolved at run time. A null member means "not available". */
struct DriverApi {
  CUresult (*StreamWriteValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int) = nullptr;
  CUresult (*StreamWaitValue32)(CUstream, CUdeviceptr, cuuint32_t, unsigned int) = nullptr;
  CUresult (*GetErrorName)(CUresult, const char**) = nullptr;
  CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
  CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
  CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
  CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
  CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
  CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
  CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
  CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
  CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
  CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
  CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
  CUresult (*MemGetAddressRange)(CUdeviceptr*, size_t*, CUdeviceptr) = nullptr;
  CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
  CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
  CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
  CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
  CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
};

/** Resolve (once) and return the table; entries stay null when no driver is present. */
const DriverApi& drv();
const char* drv_error_name(CUresult r);

/** True when a usable CUDA device exists in this process. Never throws. */
bool device_usable();

/** Create the internal stream pool and preallocate pinned flag lines. */
void init();
void finalize();
bool initialized();

/** Whether cuStreamWriteValue32 / cuStreamWaitValue32 can be used (always on CUDA >= 12 devices). */
bool stream_memory_operations_supported();

}  // namespace cuda
}  // namespace internal
}  // namespace Al
