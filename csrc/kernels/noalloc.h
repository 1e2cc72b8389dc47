// Allocation-free AllReduce over buffers that live on ONE GPU.
//
// This entry point has no counterpart in the reference library.
//
// Who it is for: callers that hold several same-sized buffers on one device
// (per-micro-batch gradient replicas, per-expert partial results, the virtual
// ranks of a single-process test) and must combine them from a place where
// device memory cannot be allocated or freed: inside a region where the
// framework's allocator is locked or its pool is exhausted on purpose, in a
// library that promised its host application a fixed memory footprint, or in
// code that runs while the driver refuses allocation calls (for instance while
// another thread captures a stream in global capture mode).  Those callers
// cannot use mncclEmuCreate / mncclEmuCollective, which cudaMalloc the control
// segments, inboxes and the parameter table.
//
// What it does: the same one-shot kernel (push into per-source inboxes, one
// barrier per block, every virtual rank reduces all contributions in rank
// order), launched once, cooperatively, over all virtual ranks.  The scratch it
// needs (barrier words, per-rank state, inboxes) sits in a file-scope
// `static __device__` array inside the library, kNoAllocScratchBytes large,
// which every GPU that loads the library holds until the process exits.  The
// kernel parameters travel by value.  No cudaMalloc, cudaFree or allocating
// library routine is called, in set-up or later.
//
// Limits (requests beyond them are rejected with ncclInvalidArgument and a
// message): 2..kNoAllocMaxRanks buffers, at most kNoAllocMaxBytes bytes each;
// types fp32, fp16, bf16, int32; operators sum, prod, max, min, avg.
//
// First call on a device: looks up the device address of the scratch array
// (cudaGetSymbolAddress, with that device current) and keeps it; make that
// first call outside of any stream capture.
//
// Sharing: every call on a device uses the same array.  Each call first clears
// the barrier words and per-rank state on `stream`, so it does not depend on
// what the previous call left behind (a call that was aborted, say); the
// inboxes are not cleared, they are always written before they are read.  Two
// calls that overlap on the GPU (different streams, no ordering between them)
// race on the array; order them.
#pragma once
#include <stddef.h>

#include "mini_nccl_api.h"

#ifdef __cplusplus
extern "C" {
#endif

enum { kNoAllocMaxRanks = 4 };
enum { kNoAllocMaxBytes = 64 * 1024 };

/* recv[r][i] = scale-free reduction over r' of send[r'][i], for every r.
 * send / recv: `nbuffers` device pointers each (host arrays of pointers); send[r] may equal recv[r]. */
ncclResult_t mncclLocalAllReduceNoAlloc(const void* const* send, void* const* recv, int nbuffers, size_t count,
                                        ncclDataType_t datatype, ncclRedOp_t op, cudaStream_t stream);

/* Size in bytes of the static scratch array (per GPU). */
size_t mncclNoAllocScratchBytes(void);

/* Outcome of the last call on the current device: *status 0 when every wait inside its kernel completed,
 * 1 when one ran out of its two-second budget, 2 when it was aborted; *detail (may be NULL) names the
 * block and the virtual rank that was waited for.  A call whose kernel gave up returns ncclSuccess all
 * the same and leaves its output incomplete, so a caller that cannot tolerate that asks here.
 * Synchronises `stream`, reads a few bytes of the scratch, allocates nothing. */
ncclResult_t mncclNoAllocLastStatus(cudaStream_t stream, unsigned* status, unsigned* detail);

#ifdef __cplusplus
}
#endif
