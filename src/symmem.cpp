// Symmetric device memory and topology discovery (see al/device/symmem.hpp).
#include "al/device/symmem.hpp"

#include <fcntl.h>
#include <unistd.h>

#include <sstream>

#include "al/tuning.hpp"
#include "al/util/meta.hpp"
#include "al/util/utils.hpp"

namespace Al {
namespace internal {
namespace device {

namespace {

bool drv_has_vmm() {
  const auto& d = cuda::drv();
  return d.MemCreate && d.MemRelease && d.MemAddressReserve && d.MemAddressFree && d.MemMap && d.MemUnmap &&
         d.MemSetAccess && d.MemExportToShareableHandle && d.MemImportFromShareableHandle &&
         d.MemGetAllocationGranularity && d.DeviceGet && d.DeviceGetAttribute;
}
bool drv_has_multicast() {
  const auto& d = cuda::drv();
  return d.MulticastCreate && d.MulticastAddDevice && d.MulticastBindMem && d.MulticastGetGranularity;
}

int device_attr(CUdevice_attribute a, int dev) {
  const auto& d = cuda::drv();
  if (!d.DeviceGet || !d.DeviceGetAttribute) return 0;
  CUdevice cd;
  int v = 0;
  if (d.DeviceGet(&cd, dev) != CUDA_SUCCESS) return 0;
  if (d.DeviceGetAttribute(&v, a, cd) != CUDA_SUCCESS) return 0;
  return v;
}

/** All ranks learn whether every rank succeeded. */
bool all_ok(const Group& g, bool mine) {
  std::vector<char> flags((size_t)g.size());
  char m = mine ? 1 : 0;
  g.allgather(&m, flags.data(), 1);
  for (char f : flags)
    if (!f) return false;
  return true;
}

CUmemAccessDesc rw_access(int dev) {
  CUmemAccessDesc a{};
  a.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  a.location.id = dev;
  a.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  return a;
}

}  // namespace

std::unique_ptr<SymmBlock> SymmBlock::create_emulated(int p, size_t bytes) {
  if (p < 1 || p > kMaxRanks) throw_al_exception("emulated group size must be in [1, ", kMaxRanks, "]");
  std::unique_ptr<SymmBlock> b(new SymmBlock());
  b->p_ = p;
  b->bytes_ = bytes;
  b->backing_ = "emulated";
  for (int r = 0; r < p; ++r) {
    void* ptr = nullptr;
    AL_CHECK_CUDA(cudaMalloc(&ptr, bytes));
    AL_CHECK_CUDA(cudaMemset(ptr, 0, bytes));
    b->owned_.push_back(ptr);
    b->peer_[r] = ptr;
  }
  AL_CHECK_CUDA(cudaDeviceSynchronize());
  return b;
}

std::unique_ptr<SymmBlock> SymmBlock::create(const Group& group, size_t bytes, bool want_multicast) {
  if (group.size() > kMaxRanks)
    throw_al_exception("device communicators support at most ", kMaxRanks, " ranks (one NVLink domain)");
  std::unique_ptr<SymmBlock> b(new SymmBlock());
  b->p_ = group.size();
  b->me_ = group.rank();
  b->bytes_ = bytes;
  AL_CHECK_CUDA(cudaGetDevice(&b->device_));
  const std::string mode = env_str("AL_DEV_SYMM", "vmm");
  bool done = false;
  if (mode != "ipc") done = b->try_vmm(group, bytes, want_multicast);
  if (!done) b->make_ipc(group, bytes);
  // Zero the local copy, then make sure every rank did before anyone uses it.
  AL_CHECK_CUDA(cudaMemset(b->peer_[b->me_], 0, bytes));
  AL_CHECK_CUDA(cudaDeviceSynchronize());
  group.barrier();
  return b;
}

bool SymmBlock::try_vmm(const Group& group, size_t bytes, bool want_multicast) {
  const auto& d = cuda::drv();
  bool ok = drv_has_vmm() &&
            device_attr(CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, device_) != 0;
  if (!all_ok(group, ok)) return false;

  CUmemAllocationProp prop{};
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  ok = d.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && gran > 0;

  // Multicast needs the size to be a multiple of its own granularity.
  bool mc_possible = want_multicast && tuning().dev_enable_nvls && p_ > 1 && drv_has_multicast() &&
                     device_attr(CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device_) != 0;
  mc_possible = all_ok(group, mc_possible);
  size_t mc_gran = 0;
  CUmulticastObjectProp mp{};
  if (mc_possible && ok) {
    mp.numDevices = (unsigned)p_;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mp.size = round_up(bytes, gran);
    if (d.MulticastGetGranularity(&mc_gran, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED) != CUDA_SUCCESS || mc_gran == 0)
      mc_possible = false;
  }
  mc_possible = all_ok(group, mc_possible);
  size_t size = ok ? round_up(bytes, gran) : 0;
  if (mc_possible) size = round_up(size, mc_gran);

  CUmemGenericAllocationHandle mine = 0;
  int fd = -1;
  if (ok) ok = d.MemCreate(&mine, size, &prop, 0) == CUDA_SUCCESS;
  if (ok) ok = d.MemExportToShareableHandle(&fd, mine, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS;
  if (!all_ok(group, ok)) {
    if (fd >= 0) ::close(fd);
    if (mine) d.MemRelease(mine);
    return false;
  }
  std::vector<int> fds = group.allgather_fd(fd);
  ::close(fd);

  handles_.assign((size_t)p_, 0);
  CUmemAccessDesc acc = rw_access(device_);
  for (int r = 0; r < p_ && ok; ++r) {
    CUmemGenericAllocationHandle h = mine;
    if (r != me_)
      ok = d.MemImportFromShareableHandle(&h, (void*)(uintptr_t)fds[(size_t)r], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
    if (!ok) break;
    handles_[(size_t)r] = h;
    CUdeviceptr va = 0;
    ok = d.MemAddressReserve(&va, size, mc_possible ? mc_gran : gran, 0, 0) == CUDA_SUCCESS;
    if (ok) ok = d.MemMap(va, size, 0, h, 0) == CUDA_SUCCESS;
    if (ok) ok = d.MemSetAccess(va, size, &acc, 1) == CUDA_SUCCESS;
    if (ok) peer_[r] = (void*)va;
  }
  for (int f : fds)
    if (f >= 0) ::close(f);
  if (!all_ok(group, ok))
    throw_al_exception("mapping peer memory failed on some rank (peer-to-peer access between the GPUs is required)");
  mapped_bytes_ = size;
  backing_ = "vmm";

  // ---- multicast alias ---------------------------------------------------------
  if (mc_possible) {
    mp.size = size;
    bool mok = true;
    int mfd = -1;
    if (me_ == 0) {
      mok = d.MulticastCreate(&mc_handle_, &mp) == CUDA_SUCCESS;
      if (mok) mok = d.MemExportToShareableHandle(&mfd, mc_handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) == CUDA_SUCCESS;
    }
    char root_ok = mok ? 1 : 0;
    group.bcast(&root_ok, 1, 0);
    if (root_ok) {
      // Distribute the descriptor (every rank takes part in the exchange; non-roots pass a dummy).
      int dummy = mfd >= 0 ? mfd : ::open("/dev/null", O_RDONLY | O_CLOEXEC);
      std::vector<int> mfds = group.allgather_fd(dummy);
      if (me_ != 0)
        mok = d.MemImportFromShareableHandle(&mc_handle_, (void*)(uintptr_t)mfds[0], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) == CUDA_SUCCESS;
      for (int f : mfds)
        if (f >= 0) ::close(f);
      ::close(dummy);
      CUdevice cd;
      if (mok) mok = d.DeviceGet(&cd, device_) == CUDA_SUCCESS && d.MulticastAddDevice(mc_handle_, cd) == CUDA_SUCCESS;
      mok = all_ok(group, mok);  // every device must be added before any bind
      if (mok) {
        mok = d.MulticastBindMem(mc_handle_, 0, mine, 0, size, 0) == CUDA_SUCCESS;
        mc_bound_ = mok;
      }
      mok = all_ok(group, mok);
      if (mok) {
        CUdeviceptr va = 0;
        mok = d.MemAddressReserve(&va, size, mc_gran, 0, 0) == CUDA_SUCCESS;
        if (mok) mok = d.MemMap(va, size, 0, mc_handle_, 0) == CUDA_SUCCESS;
        if (mok) mok = d.MemSetAccess(va, size, &acc, 1) == CUDA_SUCCESS;
        if (mok) mc_ = (void*)va;
      }
      if (!all_ok(group, mok)) mc_ = nullptr;
    }
  }
  return true;
}

void SymmBlock::make_ipc(const Group& group, size_t bytes) {
  void* mine = nullptr;
  AL_CHECK_CUDA(cudaMalloc(&mine, bytes));
  owned_.push_back(mine);
  cudaIpcMemHandle_t h;
  AL_CHECK_CUDA(cudaIpcGetMemHandle(&h, mine));
  std::vector<cudaIpcMemHandle_t> all((size_t)p_);
  group.allgather(&h, all.data(), sizeof(h));
  for (int r = 0; r < p_; ++r) {
    if (r == me_) { peer_[r] = mine; continue; }
    void* ptr = nullptr;
    AL_CHECK_CUDA(cudaIpcOpenMemHandle(&ptr, all[(size_t)r], cudaIpcMemLazyEnablePeerAccess));
    ipc_opened_.push_back(ptr);
    peer_[r] = ptr;
  }
  backing_ = "ipc";
}

SymmBlock::~SymmBlock() {
  const auto& d = cuda::drv();
  if (mc_ && d.MemUnmap) {
    d.MemUnmap((CUdeviceptr)mc_, mapped_bytes_);
    d.MemAddressFree((CUdeviceptr)mc_, mapped_bytes_);
  }
  if (mc_handle_) {
    CUdevice cd;
    if (mc_bound_ && d.MulticastUnbind && d.DeviceGet(&cd, device_) == CUDA_SUCCESS)
      d.MulticastUnbind(mc_handle_, cd, 0, mapped_bytes_);
    d.MemRelease(mc_handle_);
  }
  if (!handles_.empty()) {
    for (int r = 0; r < p_; ++r) {
      if (peer_[r]) {
        d.MemUnmap((CUdeviceptr)peer_[r], mapped_bytes_);
        d.MemAddressFree((CUdeviceptr)peer_[r], mapped_bytes_);
      }
      if (handles_[(size_t)r]) d.MemRelease(handles_[(size_t)r]);
    }
  }
  for (void* p : ipc_opened_) AL_WARN_CUDA(cudaIpcCloseMemHandle(p));
  for (void* p : owned_) AL_WARN_CUDA(cudaFree(p));
}

// ---------------------------------------------------------------------------

Topology discover_topology() {
  Topology t;
  if (!cuda::device_usable()) return t;
  AL_CHECK_CUDA(cudaGetDeviceCount(&t.device_count));
  AL_CHECK_CUDA(cudaGetDevice(&t.device));
  cudaDeviceProp prop;
  AL_CHECK_CUDA(cudaGetDeviceProperties(&prop, t.device));
  t.name = prop.name;
  t.sm_count = prop.multiProcessorCount;
  t.cc_major = prop.major;
  t.cc_minor = prop.minor;
  t.total_mem = prop.totalGlobalMem;
  t.multicast_supported = drv_has_multicast() && device_attr(CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, t.device) != 0;
  t.vmm_fd_supported =
      drv_has_vmm() && device_attr(CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, t.device) != 0;
  for (int i = 0; i < t.device_count; ++i) {
    int acc = i == t.device, atom = i == t.device;
    if (i != t.device) {
      if (cudaDeviceGetP2PAttribute(&acc, cudaDevP2PAttrAccessSupported, t.device, i) != cudaSuccess) { acc = 0; (void)cudaGetLastError(); }
      if (cudaDeviceGetP2PAttribute(&atom, cudaDevP2PAttrNativeAtomicSupported, t.device, i) != cudaSuccess) { atom = 0; (void)cudaGetLastError(); }
    }
    t.p2p_access.push_back(acc);
    t.p2p_native_atomics.push_back(atom);
  }
  return t;
}

std::string Topology::describe() const {
  std::ostringstream ss;
  if (device_count == 0) { ss << "no CUDA device usable\n"; return ss.str(); }
  ss << "devices visible: " << device_count << "\n"
     << "current device: " << device << " (" << name << ", sm_" << cc_major << cc_minor << ", " << sm_count
     << " SMs, " << (total_mem >> 20) << " MiB)\n"
     << "multicast (NVLS) supported: " << (multicast_supported ? "yes" : "no") << "\n"
     << "shareable VMM handles (posix fd): " << (vmm_fd_supported ? "yes" : "no") << "\n"
     << "peer access from current device:";
  for (int i = 0; i < device_count; ++i) ss << " " << i << ":" << (p2p_access[(size_t)i] ? "y" : "n");
  ss << "\npeer native atomics:";
  for (int i = 0; i < device_count; ++i) ss << " " << i << ":" << (p2p_native_atomics[(size_t)i] ? "y" : "n");
  ss << "\n";
  return ss.str();
}

}  // namespace device
}  // namespace internal
}  // namespace Al
