// C ABI bridge.  Every entry point checks its arguments, runs the C++ core
// inside try / catch and converts any exception into an ncclResult_t, so no
// exception crosses the ABI: the reference's "exception firewall" (reference:
// src/api.cpp:28-66,136-190).  Mapping: Error carries its own code; other
// std::exception -> ncclSystemError at init (as the reference) and
// ncclInternalError elsewhere; anything else -> ncclSystemError.
//
// Unlike the reference, ncclAllReduce is asynchronous with respect to the
// stream (the reference's watchdog loop blocks the caller until the stream is
// idle, reference: src/mini_nccl.cu:200-216); MINI_NCCL_BLOCKING=1 restores
// the blocking behaviour.  Out-of-place calls need no pre-copy (reference:
// src/api.cpp:173-175): the kernels read sendbuff and write recvbuff.
#include "mini_nccl_api.h"

#include <cstring>
#include <exception>
#include <string>

#include "comm.h"
#include "core/log.h"
#include "core/nvtx.h"

using mnccl::Comm;
using mnccl::DType;
using mnccl::RedOp;
using mnccl::Result;

namespace {

inline ncclResult_t to_c(Result r) { return static_cast<ncclResult_t>(static_cast<int>(r)); }
inline Comm* unwrap(ncclComm_t c) { return reinterpret_cast<Comm*>(c); }

template <typename Fn>
ncclResult_t firewall(const char* where, ncclResult_t std_exception_code, Fn&& fn) {
  try {
    fn();
    return ncclSuccess;
  } catch (const mnccl::Error& e) {
    if (e.code() != Result::InvalidArgument) mnccl::log_always("Mini-NCCL", "%s failed: %s", where, e.what());
    else MNCCL_INFO("Mini-NCCL", "%s: %s", where, e.what());
    return to_c(e.code());
  } catch (const std::exception& e) {
    mnccl::log_always("Mini-NCCL", "%s failed: %s", where, e.what());
    return std_exception_code;
  } catch (...) {
    mnccl::log_always("Mini-NCCL", "%s failed: unknown exception", where);
    return ncclSystemError;
  }
}

}  // namespace

extern "C" {

#define MNCCL_EXPORT __attribute__((visibility("default")))

MNCCL_EXPORT const char* mncclGetErrorString(ncclResult_t result) {
  switch (result) {
    case ncclSuccess: return "no error";
    case ncclUnhandledCudaError: return "unhandled cuda error";
    case ncclSystemError: return "system error";
    case ncclInternalError: return "internal error";
    case ncclInvalidArgument: return "invalid argument";
    case ncclInvalidUsage: return "invalid usage";
    case ncclRemoteError: return "remote error";
    case ncclInProgress: return "in progress";
    default: return "unknown error";
  }
}

MNCCL_EXPORT ncclResult_t mncclCommInitRank(ncclComm_t* comm, int nRanks, int rank, const char* ip) {
  if (!comm) return ncclInvalidArgument;
  *comm = nullptr;
  if (rank != -1 && (nRanks <= 0 || rank < 0 || rank >= nRanks)) return ncclInvalidArgument;
  mnccl::NvtxRange range("mini_ncclCommInitRank", 0xFF00A0FF, static_cast<uint64_t>(nRanks));
  return firewall("Init", ncclSystemError, [&] { *comm = reinterpret_cast<ncclComm_t>(Comm::create(nRanks, rank, ip)); });
}

MNCCL_EXPORT ncclResult_t mncclCommDestroy(ncclComm_t comm) {
  if (!comm) return ncclInvalidArgument;
  return firewall("Destroy", ncclInternalError, [&] { delete unwrap(comm); });
}

MNCCL_EXPORT ncclResult_t mncclCommUserRank(const ncclComm_t comm, int* rank) {
  if (!comm || !rank) return ncclInvalidArgument;
  return firewall("UserRank", ncclInternalError, [&] { *rank = unwrap(comm)->rank(); });
}

MNCCL_EXPORT ncclResult_t mncclCommCount(const ncclComm_t comm, int* count) {
  if (!comm || !count) return ncclInvalidArgument;
  return firewall("Count", ncclInternalError, [&] { *count = unwrap(comm)->size(); });
}

MNCCL_EXPORT ncclResult_t mncclAllReduceEx(const void* sendbuff, ncclDataType_t send_type, void* recvbuff,
                                           ncclDataType_t recv_type, ncclDataType_t wire_type, size_t count,
                                           ncclRedOp_t op, double scale, mncclAlgo_t algo, ncclComm_t comm,
                                           cudaStream_t stream) {
  if (!comm || !sendbuff || !recvbuff) return ncclInvalidArgument;
  if (!mnccl::valid_dtype(send_type) || !mnccl::valid_dtype(recv_type) || !mnccl::valid_dtype(wire_type) ||
      !mnccl::valid_op(op) || algo < mncclAlgoAuto || algo > mncclAlgoPipe || algo == mncclAlgoLocal)
    return ncclInvalidArgument;
  if (count == 0) return ncclSuccess;
  // One range per call, named and coloured as in the reference; the payload is
  // the element count.  Popped on every exit path by the destructor.
  mnccl::NvtxRange range("mini_ncclAllReduce", 0xFFFF0000, static_cast<uint64_t>(count));
  return firewall("AllReduce", ncclInternalError, [&] {
    unwrap(comm)->all_reduce(sendbuff, static_cast<DType>(send_type), recvbuff, static_cast<DType>(recv_type),
                             static_cast<DType>(wire_type), count, static_cast<RedOp>(op), scale,
                             static_cast<mnccl::Algo>(algo), stream);
  });
}

MNCCL_EXPORT ncclResult_t mncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
                                         ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  return mncclAllReduceEx(sendbuff, datatype, recvbuff, datatype, datatype, count, op, 1.0, mncclAlgoAuto, comm, stream);
}

MNCCL_EXPORT ncclResult_t mncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount,
                                             ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm,
                                             cudaStream_t stream) {
  if (!comm || !sendbuff || !recvbuff) return ncclInvalidArgument;
  if (!mnccl::valid_dtype(datatype) || !mnccl::valid_op(op)) return ncclInvalidArgument;
  if (recvcount == 0) return ncclSuccess;
  mnccl::NvtxRange range("mini_ncclReduceScatter", 0xFFFF8000, static_cast<uint64_t>(recvcount));
  return firewall("ReduceScatter", ncclInternalError, [&] {
    unwrap(comm)->reduce_scatter(sendbuff, recvbuff, recvcount, static_cast<DType>(datatype), static_cast<RedOp>(op), stream);
  });
}

MNCCL_EXPORT ncclResult_t mncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount,
                                         ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream) {
  if (!comm || !sendbuff || !recvbuff) return ncclInvalidArgument;
  if (!mnccl::valid_dtype(datatype)) return ncclInvalidArgument;
  if (sendcount == 0) return ncclSuccess;
  mnccl::NvtxRange range("mini_ncclAllGather", 0xFFFFC000, static_cast<uint64_t>(sendcount));
  return firewall("AllGather", ncclInternalError, [&] {
    unwrap(comm)->all_gather(sendbuff, recvbuff, sendcount, static_cast<DType>(datatype), stream);
  });
}

MNCCL_EXPORT ncclResult_t mncclMemAlloc(ncclComm_t comm, size_t bytes, void** ptr) {
  if (!comm || !ptr || bytes == 0) return ncclInvalidArgument;
  *ptr = nullptr;
  return firewall("MemAlloc", ncclInternalError, [&] { *ptr = unwrap(comm)->mem_alloc(bytes); });
}

MNCCL_EXPORT ncclResult_t mncclMemFree(ncclComm_t comm, void* ptr) {
  if (!comm || !ptr) return ncclInvalidArgument;
  return firewall("MemFree", ncclInternalError, [&] { unwrap(comm)->mem_free(ptr); });
}

MNCCL_EXPORT ncclResult_t mncclMemPeerPointers(ncclComm_t comm, void* ptr, void** peer_ptrs, void** mc_ptr) {
  if (!comm || !ptr || !peer_ptrs) return ncclInvalidArgument;
  return firewall("MemPeerPointers", ncclInternalError, [&] { unwrap(comm)->peer_pointers(ptr, peer_ptrs, mc_ptr); });
}

MNCCL_EXPORT ncclResult_t mncclCommRegister(ncclComm_t comm, void* buff, size_t bytes) {
  if (!comm || !buff || bytes == 0) return ncclInvalidArgument;
  return firewall("Register", ncclInternalError, [&] { unwrap(comm)->register_buffer(buff, bytes); });
}

MNCCL_EXPORT ncclResult_t mncclCommDeregister(ncclComm_t comm, void* buff) {
  if (!comm || !buff) return ncclInvalidArgument;
  return firewall("Deregister", ncclInternalError, [&] { unwrap(comm)->deregister_buffer(buff); });
}

MNCCL_EXPORT ncclResult_t mncclBarrier(ncclComm_t comm) {
  if (!comm) return ncclInvalidArgument;
  return firewall("Barrier", ncclInternalError, [&] { unwrap(comm)->barrier(); });
}

MNCCL_EXPORT ncclResult_t mncclCommAbort(ncclComm_t comm) {
  if (!comm) return ncclInvalidArgument;
  return firewall("Abort", ncclInternalError, [&] { unwrap(comm)->abort(); });
}

MNCCL_EXPORT ncclResult_t mncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* async_error) {
  if (!comm || !async_error) return ncclInvalidArgument;
  return firewall("GetAsyncError", ncclInternalError, [&] { *async_error = to_c(unwrap(comm)->async_error()); });
}

MNCCL_EXPORT ncclResult_t mncclCommStats(ncclComm_t comm, char* buf, size_t len) {
  if (!comm || !buf || len == 0) return ncclInvalidArgument;
  return firewall("Stats", ncclInternalError, [&] {
    std::string s = unwrap(comm)->stats_json();
    size_t n = s.size() < len - 1 ? s.size() : len - 1;
    memcpy(buf, s.data(), n);
    buf[n] = '\0';
  });
}

MNCCL_EXPORT ncclResult_t mncclCommQueryAlgo(ncclComm_t comm, size_t bytes, ncclDataType_t datatype, ncclRedOp_t op,
                                             int registered, mncclAlgo_t* algo) {
  if (!comm || !algo || !mnccl::valid_dtype(datatype) || !mnccl::valid_op(op)) return ncclInvalidArgument;
  return firewall("QueryAlgo", ncclInternalError, [&] {
    *algo = static_cast<mncclAlgo_t>(unwrap(comm)->query_algo(bytes, static_cast<DType>(datatype), static_cast<RedOp>(op), registered != 0));
  });
}

MNCCL_EXPORT ncclResult_t mncclCommDeviceHandle(ncclComm_t comm, void* out, size_t len, size_t* needed) {
  if (!comm) return ncclInvalidArgument;
  if (needed) *needed = sizeof(mnccl::CommDev);
  if (out && len) {
    const mnccl::CommDev& d = unwrap(comm)->device_handle();
    memcpy(out, &d, len < sizeof(d) ? len : sizeof(d));
  }
  return ncclSuccess;
}

MNCCL_EXPORT ncclResult_t mncclCommSetTuning(ncclComm_t comm, int max_blocks, int unroll) {
  if (!comm || max_blocks < 0 || max_blocks > mnccl::kMaxBlocks || (unroll != 0 && unroll != 4 && unroll != 8)) return ncclInvalidArgument;
  return firewall("SetTuning", ncclInternalError, [&] { unwrap(comm)->set_tuning(max_blocks, unroll); });
}

MNCCL_EXPORT ncclResult_t mncclCommSetKnob(ncclComm_t comm, const char* name, long long value) {
  if (!comm || !name) return ncclInvalidArgument;
  ncclResult_t bad = ncclSuccess;
  ncclResult_t r = firewall("SetKnob", ncclInternalError, [&] {
    if (!unwrap(comm)->set_knob(name, value)) bad = ncclInvalidArgument;
  });
  return r != ncclSuccess ? r : bad;
}

MNCCL_EXPORT unsigned mncclVersion(void) { return 101; }

// ---- reference-compatible names -------------------------------------------
// Linked with -Bsymbolic-functions, so these never resolve to another NCCL in
// the process, and a process that has the real NCCL loaded should bind to the
// mnccl* names instead.

MNCCL_EXPORT const char* ncclGetErrorString(ncclResult_t r) { return mncclGetErrorString(r); }
MNCCL_EXPORT ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nRanks, int rank, const char* ip) {
  return mncclCommInitRank(comm, nRanks, rank, ip);
}
MNCCL_EXPORT ncclResult_t ncclCommDestroy(ncclComm_t comm) { return mncclCommDestroy(comm); }
MNCCL_EXPORT ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank) { return mncclCommUserRank(comm, rank); }
MNCCL_EXPORT ncclResult_t ncclCommCount(const ncclComm_t comm, int* count) { return mncclCommCount(comm, count); }
MNCCL_EXPORT ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count, ncclDataType_t datatype,
                                        ncclRedOp_t op, ncclComm_t comm, cudaStream_t stream) {
  return mncclAllReduce(sendbuff, recvbuff, count, datatype, op, comm, stream);
}

}  // extern "C"
