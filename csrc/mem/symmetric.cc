#include "mem/symmetric.h"

#include <cuda_runtime.h>
#include <unistd.h>

#include <cstring>

#include "bootstrap/fdpass.h"
#include "bootstrap/store.h"
#include "core/error.h"
#include "core/log.h"
#include "mem/cuda_driver.h"

namespace mnccl {

struct Segment::Impl {
  bool vmm = false;
  int nranks = 0;
  int rank = 0;
  size_t mapped = 0;
  // vmm
  std::vector<CUmemGenericAllocationHandle> handles;  // per rank (own at [rank])
  std::vector<CUdeviceptr> vas;
  CUmemGenericAllocationHandle mc_handle = 0;
  CUdeviceptr mc_va = 0;
  bool mc_bound = false;
  int device = 0;
  // ipc
  void* ipc_own = nullptr;
  std::vector<void*> ipc_peer;

  ~Impl() {
    const CudaDriver* d = CudaDriver::get();
    if (vmm && d) {
      if (mc_va) {
        d->MemUnmap(mc_va, mapped);
        d->MemAddressFree(mc_va, mapped);
      }
      if (mc_handle) {
        if (mc_bound) d->MulticastUnbind(mc_handle, device, 0, mapped);
        d->MemRelease(mc_handle);
      }
      for (size_t r = 0; r < vas.size(); ++r) {
        if (vas[r]) {
          d->MemUnmap(vas[r], mapped);
          d->MemAddressFree(vas[r], mapped);
        }
      }
      for (size_t r = 0; r < handles.size(); ++r)
        if (handles[r]) d->MemRelease(handles[r]);
    } else if (!vmm) {
      for (size_t r = 0; r < ipc_peer.size(); ++r)
        if (ipc_peer[r] && static_cast<int>(r) != rank) cudaIpcCloseMemHandle(ipc_peer[r]);
      if (ipc_own) cudaFree(ipc_own);
    }
  }
};

namespace {

#define DRV_TRY(d, call, what)                                                                 \
  do {                                                                                         \
    CUresult _r = (call);                                                                      \
    if (_r != CUDA_SUCCESS) fail(Result::UnhandledCudaError, std::string(what) + ": " + (d)->error_string(_r)); \
  } while (0)

#define RT_TRY(call, what)                                                                     \
  do {                                                                                         \
    cudaError_t _e = (call);                                                                   \
    if (_e != cudaSuccess) {                                                                   \
      (void)cudaGetLastError();                                                                \
      fail(Result::UnhandledCudaError, std::string(what) + ": " + cudaGetErrorString(_e));     \
    }                                                                                          \
  } while (0)

size_t round_up(size_t x, size_t g) { return (x + g - 1) / g * g; }

int dev_attr(const CudaDriver* d, CUdevice_attribute a, int device) {
  CUdevice dev;
  int v = 0;
  if (d->DeviceGet(&dev, device) != CUDA_SUCCESS) return 0;
  if (d->DeviceGetAttribute(&v, a, dev) != CUDA_SUCCESS) return 0;
  return v;
}

}  // namespace

bool SymmetricMemory::all_agree(bool mine) {
  uint8_t m = mine ? 1 : 0;
  std::vector<uint8_t> all(size_);
  store_->all_gather(&m, all.data(), 1);
  for (uint8_t v : all)
    if (!v) return false;
  return true;
}

SymmetricMemory::SymmetricMemory(int rank, int size, int device, BootstrapStore* store, FdChannel* fds,
                                 const Config& cfg)
    : rank_(rank), size_(size), device_(device), store_(store), fds_(fds), cfg_(cfg) {
  const CudaDriver* d = CudaDriver::get();
  bool vmm_ok = d && d->has_vmm && fds_ != nullptr && cfg.symm_mode != "ipc" &&
                dev_attr(d, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, device) != 0 &&
                dev_attr(d, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, device) != 0;
  bool mc_ok = vmm_ok && d->has_multicast && cfg.nvls_enable && size > 1 &&
               dev_attr(d, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, device) != 0;
  use_vmm_ = all_agree(vmm_ok);
  use_mc_ = use_vmm_ && all_agree(mc_ok);
  if (cfg.symm_mode == "vmm" && !use_vmm_) fail(Result::SystemError, "MINI_NCCL_SYMM=vmm but VMM sharing is unavailable");
  MNCCL_INFO("Mini-NCCL", "rank %d: symmetric memory provider=%s nvls=%d", rank_, provider(), use_mc_ ? 1 : 0);
}

SymmetricMemory::~SymmetricMemory() = default;

std::shared_ptr<Segment> SymmetricMemory::allocate(size_t bytes, bool want_multicast) {
  if (bytes == 0) fail(Result::InvalidArgument, "symmetric allocation of zero bytes");
  // Everyone must ask for the same size.
  uint64_t mine = bytes;
  std::vector<uint64_t> all(size_);
  store_->all_gather(&mine, all.data(), sizeof(mine));
  for (uint64_t v : all)
    if (v != mine) fail(Result::InvalidUsage, "symmetric allocation sizes differ between ranks");
  std::shared_ptr<Segment> seg;
  std::string err;
  try {
    seg = use_vmm_ ? allocate_vmm(bytes, want_multicast && use_mc_) : allocate_ipc(bytes);
  } catch (const std::exception& e) {
    err = e.what();
  }
  if (!all_agree(seg != nullptr)) {
    seg.reset();
    fail(Result::UnhandledCudaError, "symmetric allocation failed on at least one rank" + (err.empty() ? "" : (": " + err)));
  }
  seg->id = next_id_++;
  RT_TRY(cudaMemset(seg->local, 0, seg->mapped_bytes), "cudaMemset(symmetric segment)");
  RT_TRY(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  store_->barrier();
  return seg;
}

void SymmetricMemory::release(const std::shared_ptr<Segment>& seg) {
  if (!seg) return;
  cudaDeviceSynchronize();
  store_->barrier();  // nobody touches a peer's copy after this point
  seg->impl.reset();
  seg->local = nullptr;
  seg->mc = nullptr;
  seg->peer.clear();
  store_->barrier();
}

std::shared_ptr<Segment> SymmetricMemory::allocate_vmm(size_t bytes, bool want_mc) {
  const CudaDriver* d = CudaDriver::get();
  auto seg = std::make_shared<Segment>();
  auto impl = std::make_shared<Segment::Impl>();
  seg->impl = impl;
  impl->vmm = true;
  impl->nranks = size_;
  impl->rank = rank_;
  impl->device = device_;
  impl->handles.assign(size_, 0);
  impl->vas.assign(size_, 0);

  CUmemAllocationProp prop;
  memset(&prop, 0, sizeof(prop));
  prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
  prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  prop.location.id = device_;
  prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
  size_t gran = 0;
  DRV_TRY(d, d->MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
  CUmulticastObjectProp mcprop;
  memset(&mcprop, 0, sizeof(mcprop));
  bool mc = want_mc;
  if (mc) {
    mcprop.numDevices = static_cast<unsigned>(size_);
    mcprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    mcprop.size = round_up(bytes, gran);
    size_t mgran = 0;
    if (d->MulticastGetGranularity(&mgran, &mcprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mgran)
      gran = gran > mgran ? gran : mgran;
    else
      mc = false;
  }
  // The multicast decision must be identical everywhere before sizes are fixed.
  mc = all_agree(mc);
  const size_t mapped = round_up(bytes, gran);
  impl->mapped = mapped;
  mcprop.size = mapped;

  DRV_TRY(d, d->MemCreate(&impl->handles[rank_], mapped, &prop, 0), "cuMemCreate");
  int my_fd = -1;
  DRV_TRY(d, d->MemExportToShareableHandle(&my_fd, impl->handles[rank_], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
          "cuMemExportToShareableHandle");
  const uint32_t tag = next_id_ * 4u;
  const int tmo = cfg_.socket_timeout_ms;
  try {
    for (int k = 1; k < size_; ++k) fds_->send_fd((rank_ + k) % size_, my_fd, tag, tmo);
    for (int k = 1; k < size_; ++k) {
      int src = -1;
      uint32_t got_tag = 0;
      int fd = fds_->recv_fd(&src, &got_tag, tmo);
      if (src < 0 || src >= size_ || src == rank_ || got_tag != tag || impl->handles[src]) {
        ::close(fd);
        fail(Result::InternalError, "unexpected descriptor while exchanging memory handles");
      }
      CUresult r = d->MemImportFromShareableHandle(&impl->handles[src], reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                   CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
      ::close(fd);
      if (r != CUDA_SUCCESS) fail(Result::UnhandledCudaError, "cuMemImportFromShareableHandle: " + d->error_string(r));
    }
  } catch (...) {
    ::close(my_fd);
    throw;
  }
  ::close(my_fd);

  CUmemAccessDesc access;
  memset(&access, 0, sizeof(access));
  access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
  access.location.id = device_;
  access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
  seg->peer.assign(size_, nullptr);
  for (int r = 0; r < size_; ++r) {
    DRV_TRY(d, d->MemAddressReserve(&impl->vas[r], mapped, gran, 0, 0), "cuMemAddressReserve");
    DRV_TRY(d, d->MemMap(impl->vas[r], mapped, 0, impl->handles[r], 0), "cuMemMap");
    DRV_TRY(d, d->MemSetAccess(impl->vas[r], mapped, &access, 1), "cuMemSetAccess");
    seg->peer[r] = reinterpret_cast<void*>(impl->vas[r]);
  }
  seg->local = seg->peer[rank_];
  seg->bytes = bytes;
  seg->mapped_bytes = mapped;

  if (mc) {
    // Every step is attempted by every rank; agreement is checked at the
    // collective points so that no rank waits for one that gave up.
    bool ok = true;
    std::string why;
    const uint32_t mctag = tag + 1;
    if (rank_ == 0) {
      CUresult r = d->MulticastCreate(&impl->mc_handle, &mcprop);
      if (r != CUDA_SUCCESS) { ok = false; why = "cuMulticastCreate: " + d->error_string(r); impl->mc_handle = 0; }
    }
    // A gather through rank 0: nobody passes this point before every rank has
    // finished exchanging the memory descriptors above, so the multicast
    // descriptor cannot be mistaken for one of those.
    const bool created = all_agree(ok);
    if (created) {
      try {
        if (rank_ == 0) {
          int mfd = -1;
          DRV_TRY(d, d->MemExportToShareableHandle(&mfd, impl->mc_handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
                  "cuMemExportToShareableHandle(multicast)");
          try {
            for (int p = 1; p < size_; ++p) fds_->send_fd(p, mfd, mctag, tmo);
          } catch (...) { ::close(mfd); throw; }
          ::close(mfd);
        } else {
          int src = -1;
          uint32_t got_tag = 0;
          int fd = fds_->recv_fd(&src, &got_tag, tmo);
          CUresult r = CUDA_ERROR_UNKNOWN;
          if (src == 0 && got_tag == mctag)
            r = d->MemImportFromShareableHandle(&impl->mc_handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
          ::close(fd);
          if (r != CUDA_SUCCESS) { impl->mc_handle = 0; fail(Result::UnhandledCudaError, "multicast import: " + d->error_string(r)); }
        }
        CUdevice cudev;
        DRV_TRY(d, d->DeviceGet(&cudev, device_), "cuDeviceGet");
        DRV_TRY(d, d->MulticastAddDevice(impl->mc_handle, cudev), "cuMulticastAddDevice");
      } catch (const std::exception& e) {
        ok = false;
        why = e.what();
      }
    } else {
      ok = false;
    }
    ok = all_agree(ok);  // all devices added (binding before that is an error)
    if (ok) {
      CUresult r = d->MulticastBindMem(impl->mc_handle, 0, impl->handles[rank_], 0, mapped, 0);
      if (r == CUDA_SUCCESS) impl->mc_bound = true;
      else { ok = false; why = "cuMulticastBindMem: " + d->error_string(r); }
      ok = all_agree(ok);
    }
    if (ok) {
      CUresult r = d->MemAddressReserve(&impl->mc_va, mapped, gran, 0, 0);
      if (r == CUDA_SUCCESS) r = d->MemMap(impl->mc_va, mapped, 0, impl->mc_handle, 0);
      if (r == CUDA_SUCCESS) r = d->MemSetAccess(impl->mc_va, mapped, &access, 1);
      if (r != CUDA_SUCCESS) { ok = false; why = "multicast map: " + d->error_string(r); }
      ok = all_agree(ok);
    }
    if (ok) {
      seg->mc = reinterpret_cast<void*>(impl->mc_va);
    } else {
      if (!why.empty()) MNCCL_WARN("Mini-NCCL", "rank %d: NVLS disabled for this allocation (%s)", rank_, why.c_str());
      // Tear the partial multicast state down; the P2P mappings stay.
      if (impl->mc_va) { d->MemUnmap(impl->mc_va, mapped); d->MemAddressFree(impl->mc_va, mapped); impl->mc_va = 0; }
      if (impl->mc_handle) {
        if (impl->mc_bound) d->MulticastUnbind(impl->mc_handle, device_, 0, mapped);
        impl->mc_bound = false;
        d->MemRelease(impl->mc_handle);
        impl->mc_handle = 0;
      }
      use_mc_ = false;  // do not try again on later allocations
    }
  }
  return seg;
}

std::shared_ptr<Segment> SymmetricMemory::allocate_ipc(size_t bytes) {
  auto seg = std::make_shared<Segment>();
  auto impl = std::make_shared<Segment::Impl>();
  seg->impl = impl;
  impl->vmm = false;
  impl->nranks = size_;
  impl->rank = rank_;
  const size_t mapped = round_up(bytes, size_t(2) << 20);
  impl->mapped = mapped;
  RT_TRY(cudaMalloc(&impl->ipc_own, mapped), "cudaMalloc(symmetric segment)");
  cudaIpcMemHandle_t mine;
  RT_TRY(cudaIpcGetMemHandle(&mine, impl->ipc_own), "cudaIpcGetMemHandle");
  std::vector<cudaIpcMemHandle_t> all(size_);
  store_->all_gather(&mine, all.data(), sizeof(mine));
  impl->ipc_peer.assign(size_, nullptr);
  seg->peer.assign(size_, nullptr);
  for (int r = 0; r < size_; ++r) {
    if (r == rank_) {
      impl->ipc_peer[r] = impl->ipc_own;
    } else {
      RT_TRY(cudaIpcOpenMemHandle(&impl->ipc_peer[r], all[r], cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    }
    seg->peer[r] = impl->ipc_peer[r];
  }
  seg->local = impl->ipc_own;
  seg->bytes = bytes;
  seg->mapped_bytes = mapped;
  return seg;
}

}  // namespace mnccl
