// CUDA driver entry points, resolved at run time through the runtime's
// cudaGetDriverEntryPoint.  The library is linked against the static CUDA
// runtime only, so it loads (and its CPU-only network path works) on machines
// without a driver; the virtual-memory and multicast calls needed for
// symmetric memory are looked up on first use.
#pragma once
#include <cuda.h>

#include <string>

namespace mnccl {

struct CudaDriver {
  decltype(&cuGetErrorString) GetErrorString = nullptr;
  decltype(&cuDeviceGet) DeviceGet = nullptr;
  decltype(&cuDeviceGetAttribute) DeviceGetAttribute = nullptr;
  decltype(&cuMemGetAllocationGranularity) MemGetAllocationGranularity = nullptr;
  decltype(&cuMemCreate) MemCreate = nullptr;
  decltype(&cuMemRelease) MemRelease = nullptr;
  decltype(&cuMemExportToShareableHandle) MemExportToShareableHandle = nullptr;
  decltype(&cuMemImportFromShareableHandle) MemImportFromShareableHandle = nullptr;
  decltype(&cuMemAddressReserve) MemAddressReserve = nullptr;
  decltype(&cuMemAddressFree) MemAddressFree = nullptr;
  decltype(&cuMemMap) MemMap = nullptr;
  decltype(&cuMemUnmap) MemUnmap = nullptr;
  decltype(&cuMemSetAccess) MemSetAccess = nullptr;
  decltype(&cuMulticastCreate) MulticastCreate = nullptr;
  decltype(&cuMulticastAddDevice) MulticastAddDevice = nullptr;
  decltype(&cuMulticastBindMem) MulticastBindMem = nullptr;
  decltype(&cuMulticastUnbind) MulticastUnbind = nullptr;
  decltype(&cuMulticastGetGranularity) MulticastGetGranularity = nullptr;
  decltype(&cuStreamWriteValue32) StreamWriteValue32 = nullptr;
  decltype(&cuTensorMapEncodeTiled) TensorMapEncodeTiled = nullptr;
  decltype(&cuMemGetAddressRange) MemGetAddressRange = nullptr;
  decltype(&cuPointerGetAttribute) PointerGetAttribute = nullptr;

  bool has_vmm = false;        // every VMM entry point resolved
  bool has_multicast = false;  // every multicast entry point resolved

  // nullptr when no driver is present.
  static const CudaDriver* get();
  std::string error_string(CUresult r) const;
};

}  // namespace mnccl
