// CUDA support layer: driver entry points, stream / event / flag pools,
// GPUStatusFlag and GPUWait (see the headers under al/cuda/).
#include <atomic>
#include <mutex>

#include "al/cuda/cuda.hpp"
#include "al/cuda/events.hpp"
#include "al/cuda/gpu_status_flag.hpp"
#include "al/cuda/gpu_wait.hpp"
#include <cctype>
#include <string>

#include "al/cuda/helper_kernels.hpp"
#include "al/cuda/streams.hpp"
#include "al/cuda/sync_memory.hpp"
#include "al/profiling.hpp"
#include "al/tuning.hpp"

namespace Al {
namespace internal {

void pe_make_device_current(int dev) {
  if (dev >= 0) (void)cudaSetDevice(dev);
}

std::string pe_device_pci_bus_id(int dev) {
  char id[32] = {0};
  if (dev < 0 || cudaDeviceGetPCIBusId(id, (int)sizeof(id), dev) != cudaSuccess) {
    (void)cudaGetLastError();
    return std::string();
  }
  std::string s(id);
  for (char& c : s) c = (char)tolower((unsigned char)c);
  return s;
}

namespace cuda {

namespace {

template <typename Fn>
void resolve(Fn& out, const char* name) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) == cudaSuccess &&
      q == cudaDriverEntryPointSuccess)
    out = reinterpret_cast<Fn>(p);
  else
    (void)cudaGetLastError();
}

bool g_initialized = false;
bool g_memops = false;

}  // namespace

bool device_usable() {
  static const bool ok = [] {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) { (void)cudaGetLastError(); return false; }
    return n > 0;
  }();
  return ok;
}

const DriverApi& drv() {
  static const DriverApi api = [] {
    DriverApi a;
    if (!device_usable()) return a;
    resolve(a.StreamWriteValue32, "cuStreamWriteValue32");
    resolve(a.StreamWaitValue32, "cuStreamWaitValue32");
    resolve(a.GetErrorName, "cuGetErrorName");
    resolve(a.DeviceGetAttribute, "cuDeviceGetAttribute");
    resolve(a.DeviceGet, "cuDeviceGet");
    resolve(a.MemCreate, "cuMemCreate");
    resolve(a.MemRelease, "cuMemRelease");
    resolve(a.MemAddressReserve, "cuMemAddressReserve");
    resolve(a.MemAddressFree, "cuMemAddressFree");
    resolve(a.MemMap, "cuMemMap");
    resolve(a.MemUnmap, "cuMemUnmap");
    resolve(a.MemSetAccess, "cuMemSetAccess");
    resolve(a.MemExportToShareableHandle, "cuMemExportToShareableHandle");
    resolve(a.MemImportFromShareableHandle, "cuMemImportFromShareableHandle");
    resolve(a.MemGetAllocationGranularity, "cuMemGetAllocationGranularity");
    resolve(a.MemGetAddressRange, "cuMemGetAddressRange");
    resolve(a.MulticastCreate, "cuMulticastCreate");
    resolve(a.MulticastAddDevice, "cuMulticastAddDevice");
    resolve(a.MulticastBindMem, "cuMulticastBindMem");
    resolve(a.MulticastUnbind, "cuMulticastUnbind");
    resolve(a.MulticastGetGranularity, "cuMulticastGetGranularity");
    return a;
  }();
  return api;
}

const char* drv_error_name(CUresult r) {
  const char* s = nullptr;
  if (drv().GetErrorName && drv().GetErrorName(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUDA_ERROR_<unknown>";
}

// ---- pools -------------------------------------------------------------------

StreamPool stream_pool;
LockedResourcePool<cudaEvent_t, EventFactory> event_pool;
LockedResourcePool<int32_t*, SyncLineFactory> sync_pool;

void StreamPool::allocate(size_t n) {
  clear();
  int lo = 0, hi = 0;  // numerically lowest value = highest priority
  AL_CHECK_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
  for (size_t i = 0; i < n; ++i) {
    cudaStream_t s, h;
    AL_CHECK_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    AL_CHECK_CUDA(cudaStreamCreateWithPriority(&h, cudaStreamNonBlocking, hi));
    profiling::name_stream(s, "al_internal_" + std::to_string(i));
    profiling::name_stream(h, "al_internal_high_" + std::to_string(i));
    default_.push_back(s);
    high_.push_back(h);
  }
  external_ = false;
}

void StreamPool::clear() {
  if (!external_) {
    for (auto s : default_) AL_WARN_CUDA(cudaStreamDestroy(s));
    for (auto s : high_) AL_WARN_CUDA(cudaStreamDestroy(s));
  }
  default_.clear();
  high_.clear();
}

cudaStream_t StreamPool::get_stream() {
  if (default_.empty()) throw_al_exception("stream pool is empty (library not initialised with a device?)");
  return default_[next_default_.fetch_add(1, std::memory_order_relaxed) % default_.size()];
}

cudaStream_t StreamPool::get_high_priority_stream() {
  if (high_.empty()) throw_al_exception("stream pool is empty (library not initialised with a device?)");
  return high_[next_high_.fetch_add(1, std::memory_order_relaxed) % high_.size()];
}

void StreamPool::replace_streams(std::function<cudaStream_t(bool)> getter) {
  const size_t n = default_.size();
  clear();
  for (size_t i = 0; i < n; ++i) {
    default_.push_back(getter(false));
    high_.push_back(getter(true));
  }
  external_ = true;
}

namespace {
std::mutex g_slab_mu;
std::vector<void*> g_slabs;
char* g_slab_cur = nullptr;
size_t g_slab_left = 0;
constexpr size_t kSlabBytes = 64 * 1024;
}  // namespace

int32_t* SyncLineFactory::create() {
  std::lock_guard<std::mutex> g(g_slab_mu);
  if (g_slab_left < AL_DESTRUCTIVE_INTERFERENCE_SIZE) {
    void* slab = nullptr;
    AL_CHECK_CUDA(cudaHostAlloc(&slab, kSlabBytes, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(slab, 0, kSlabBytes);
    g_slabs.push_back(slab);
    g_slab_cur = (char*)slab;
    g_slab_left = kSlabBytes;
  }
  int32_t* line = (int32_t*)g_slab_cur;
  g_slab_cur += AL_DESTRUCTIVE_INTERFERENCE_SIZE;
  g_slab_left -= AL_DESTRUCTIVE_INTERFERENCE_SIZE;
  return line;
}

void SyncLineFactory::release_slabs() {
  std::lock_guard<std::mutex> g(g_slab_mu);
  for (void* s : g_slabs) AL_WARN_CUDA(cudaFreeHost(s));
  g_slabs.clear();
  g_slab_cur = nullptr;
  g_slab_left = 0;
}

// ---- init / finalize -----------------------------------------------------------

void init() {
  if (g_initialized || !device_usable()) return;
  stream_pool.allocate((size_t)std::max(1, tuning().stream_pool_size));
  // Stream memory operations are part of the baseline feature set from CUDA 12
  // on; keep the attribute probe for older drivers.
  g_memops = false;
  const auto& d = drv();
  if (d.StreamWriteValue32 && d.StreamWaitValue32) {
    int drv_ver = 0;
    AL_CHECK_CUDA(cudaDriverGetVersion(&drv_ver));
    if (drv_ver >= 12000) {
      g_memops = true;
    } else if (d.DeviceGetAttribute && d.DeviceGet) {
      int dev = 0, attr = 0;
      AL_CHECK_CUDA(cudaGetDevice(&dev));
      CUdevice cudev;
      if (d.DeviceGet(&cudev, dev) == CUDA_SUCCESS &&
          d.DeviceGetAttribute(&attr, CU_DEVICE_ATTRIBUTE_CAN_USE_STREAM_MEM_OPS_V1, cudev) == CUDA_SUCCESS)
        g_memops = attr != 0;
    }
  }
  if (getenv("AL_DISABLE_STREAM_MEM_OPS")) g_memops = false;
  sync_pool.preallocate((size_t)std::max(0, tuning().sync_mem_prealloc));
  g_initialized = true;
}

void finalize() {
  if (!g_initialized) return;
  event_pool.clear();
  sync_pool.clear();
  SyncLineFactory::release_slabs();
  stream_pool.clear();
  g_initialized = false;
}

bool initialized() { return g_initialized; }
bool stream_memory_operations_supported() { return g_memops; }

// ---- GPUStatusFlag ---------------------------------------------------------------

GPUStatusFlag::GPUStatusFlag() : use_memops_(stream_memory_operations_supported()) {
  if (use_memops_) {
    host_flag_ = sync_pool.get();
    __atomic_store_n(host_flag_, 1, __ATOMIC_SEQ_CST);  // "nothing pending" reads as complete
    void* dp = nullptr;
    AL_CHECK_CUDA(cudaHostGetDevicePointer(&dp, host_flag_, 0));
    dev_ptr_ = (CUdeviceptr)dp;
  } else {
    event_ = event_pool.get();
  }
}

GPUStatusFlag::~GPUStatusFlag() {
  if (use_memops_) sync_pool.release(host_flag_);
  else event_pool.release(event_);
}

void GPUStatusFlag::record(cudaStream_t stream) {
  if (use_memops_) {
    __atomic_store_n(host_flag_, 0, __ATOMIC_SEQ_CST);
    AL_CHECK_CUDA_DRV(drv().StreamWriteValue32((CUstream)stream, dev_ptr_, 1, CU_STREAM_WRITE_VALUE_DEFAULT));
  } else {
    AL_CHECK_CUDA(cudaEventRecord(event_, stream));
  }
}

bool GPUStatusFlag::query() {
  if (use_memops_) return __atomic_load_n(host_flag_, __ATOMIC_ACQUIRE) != 0;
  cudaError_t e = cudaEventQuery(event_);
  if (e == cudaSuccess) return true;
  if (e == cudaErrorNotReady) { (void)cudaGetLastError(); return false; }
  AL_CHECK_CUDA(e);
  return false;
}

// ---- GPUWait -------------------------------------------------------------------------

GPUWait::GPUWait() {
  host_flag_ = sync_pool.get();
  __atomic_store_n(host_flag_, 0, __ATOMIC_SEQ_CST);
  host_status_ = sync_pool.get();
  __atomic_store_n(host_status_, 0, __ATOMIC_SEQ_CST);
  void* dp = nullptr;
  AL_CHECK_CUDA(cudaHostGetDevicePointer(&dp, host_flag_, 0));
  dev_ptr_ = (CUdeviceptr)dp;
}

GPUWait::~GPUWait() {
  sync_pool.release(host_flag_);
  sync_pool.release(host_status_);
}

bool GPUWait::timed_out() const { return __atomic_load_n(host_status_, __ATOMIC_ACQUIRE) != 0; }

void GPUWait::wait(cudaStream_t stream) {
  if (stream_memory_operations_supported()) {
    launch_wait_kernel(stream, 1, dev_ptr_);
  } else {
    const uint64_t budget = (uint64_t)(tuning().dev_wait_timeout_ms * 1e6);
    void* status_dev = nullptr;
    AL_CHECK_CUDA(cudaHostGetDevicePointer(&status_dev, host_status_, 0));
    launch_wait_kernel(stream, 1, (volatile int32_t*)dev_ptr_, budget, (int32_t*)status_dev);
  }
}

void GPUWait::signal() { __atomic_store_n(host_flag_, 1, __ATOMIC_SEQ_CST); }

}  // namespace cuda
}  // namespace internal
}  // namespace Al
