// Symmetric memory: every rank allocates a segment of the same size and maps
// all peers' segments over NVLink, so a kernel can load from / store to any
// rank's copy, and (with NVLS) a multicast address that the NVSwitch fans out
// to all copies.
//
// Two providers:
//   vmm  cuMemCreate + POSIX-fd export, descriptors handed to the peers over
//        Unix sockets (SCM_RIGHTS), cuMemMap of every peer handle; optional
//        cuMulticastCreate / BindMem for NVLS.  Preferred.
//   ipc  cudaMalloc + cudaIpcGetMemHandle / OpenMemHandle.  Fallback without
//        multicast (no VMM, no fd passing).
//
// The reference attempts the same-host path with cudaIpcGetMemHandle on
// host-pinned memory, which cannot succeed, so its fast path never runs
// (reference: src/transport/RDMATransport.h:117-118,522-529,583-590); and it
// re-exchanges addresses through rank 0 on every call (:206-256).  Here the
// mapping is made once per allocation.
#pragma once
#include <cstddef>
#include <cstdint>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "core/config.h"

namespace mnccl {

class BootstrapStore;
class FdChannel;

struct Segment {
  uint32_t id = 0;
  size_t bytes = 0;          // usable bytes requested
  size_t mapped_bytes = 0;   // rounded to the granularity
  void* local = nullptr;     // this rank's copy (== peer[rank])
  std::vector<void*> peer;   // every rank's copy as mapped in this process
  void* mc = nullptr;        // multicast address or null
  // Buffers registered over CUDA IPC (mncclCommRegister): the driver's id of the allocation at the time
  // of registration (0 = not tracked).  An address range that was freed and allocated again carries
  // another id, so a stale registration is noticed before a kernel uses the peers' old mappings.
  unsigned long long buffer_id = 0;
  struct Impl;
  std::shared_ptr<Impl> impl;
};

class SymmetricMemory {
 public:
  // `device` is the CUDA device of this rank.  Collective: decides the
  // provider and NVLS availability for the whole communicator.
  SymmetricMemory(int rank, int size, int device, BootstrapStore* store, FdChannel* fds, const Config& cfg);
  ~SymmetricMemory();

  // Collective.  The segment is zero-filled.  Multicast is bound when NVLS is
  // on for this communicator and want_multicast is set; if binding fails on any
  // rank, the segment is returned without a multicast address on every rank.
  std::shared_ptr<Segment> allocate(size_t bytes, bool want_multicast);
  // Collective.
  void release(const std::shared_ptr<Segment>& seg);

  bool uses_vmm() const { return use_vmm_; }
  bool nvls_available() const { return use_mc_; }
  void disable_nvls() { use_mc_ = false; }
  const char* provider() const { return use_vmm_ ? "vmm" : "ipc"; }

 private:
  std::shared_ptr<Segment> allocate_vmm(size_t bytes, bool want_mc);
  std::shared_ptr<Segment> allocate_ipc(size_t bytes);
  bool all_agree(bool mine);

  int rank_, size_, device_;
  BootstrapStore* store_;
  FdChannel* fds_;
  Config cfg_;
  bool use_vmm_ = false, use_mc_ = false;
  uint32_t next_id_ = 1;
};

}  // namespace mnccl
