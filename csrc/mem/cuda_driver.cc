#include "mem/cuda_driver.h"

#include <cuda_runtime.h>

#include <mutex>

namespace mnccl {
namespace {

template <typename Fn>
bool resolve(const char* name, Fn* out) {
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q = cudaDriverEntryPointSymbolNotFound;
  cudaError_t e = cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q);
  if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
    (void)cudaGetLastError();
    *out = nullptr;
    return false;
  }
  *out = reinterpret_cast<Fn>(p);
  return true;
}

}  // namespace

const CudaDriver* CudaDriver::get() {
  static std::once_flag once;
  static CudaDriver* drv = nullptr;
  std::call_once(once, [] {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      return;
    }
    auto* d = new CudaDriver();
    bool base = resolve("cuGetErrorString", &d->GetErrorString) & resolve("cuDeviceGet", &d->DeviceGet) &
                resolve("cuDeviceGetAttribute", &d->DeviceGetAttribute);
    if (!base) {
      delete d;
      return;
    }
    d->has_vmm = resolve("cuMemGetAllocationGranularity", &d->MemGetAllocationGranularity) &
                 resolve("cuMemCreate", &d->MemCreate) & resolve("cuMemRelease", &d->MemRelease) &
                 resolve("cuMemExportToShareableHandle", &d->MemExportToShareableHandle) &
                 resolve("cuMemImportFromShareableHandle", &d->MemImportFromShareableHandle) &
                 resolve("cuMemAddressReserve", &d->MemAddressReserve) &
                 resolve("cuMemAddressFree", &d->MemAddressFree) & resolve("cuMemMap", &d->MemMap) &
                 resolve("cuMemUnmap", &d->MemUnmap) & resolve("cuMemSetAccess", &d->MemSetAccess);
    d->has_multicast = d->has_vmm & resolve("cuMulticastCreate", &d->MulticastCreate) &
                       resolve("cuMulticastAddDevice", &d->MulticastAddDevice) &
                       resolve("cuMulticastBindMem", &d->MulticastBindMem) &
                       resolve("cuMulticastUnbind", &d->MulticastUnbind) &
                       resolve("cuMulticastGetGranularity", &d->MulticastGetGranularity);
    resolve("cuStreamWriteValue32", &d->StreamWriteValue32);
    resolve("cuTensorMapEncodeTiled", &d->TensorMapEncodeTiled);
    resolve("cuMemGetAddressRange", &d->MemGetAddressRange);
    resolve("cuPointerGetAttribute", &d->PointerGetAttribute);
    drv = d;
  });
  return drv;
}

std::string CudaDriver::error_string(CUresult r) const {
  const char* s = nullptr;
  if (GetErrorString && GetErrorString(r, &s) == CUDA_SUCCESS && s) return s;
  return "CUDA driver error " + std::to_string(static_cast<int>(r));
}

}  // namespace mnccl
