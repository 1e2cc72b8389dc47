/*
 * mini_nccl_api.h -- public C ABI of the Blackwell-native Mini-NCCL library.
 *
 * The first block (types + six functions) is call-compatible with the reference
 * ABI (reference: include/mini_nccl_api.h:15-69): same enum values, same
 * signatures, same error strings.  Note that ncclCommInitRank takes the root /
 * master IP as a string instead of a ncclUniqueId, exactly like the reference.
 *
 * The second block ("mnccl*" names) is additive.  Every nccl* symbol has an
 * mnccl* twin with the same behaviour, so that a process that already has the
 * real libnccl loaded (a PyTorch process, for instance) can bind to this
 * library without any symbol clash.
 *
 * No C++ exception ever crosses any function declared here.
 */
#ifndef MINI_NCCL_B200_API_H_
#define MINI_NCCL_B200_API_H_

#include <stddef.h>
#include <stdint.h>

#if defined(MINI_NCCL_NO_CUDA_HEADERS)
typedef struct CUstream_st* cudaStream_t;
#else
#include <cuda_runtime.h>
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---------------------------------------------------------------- types */

typedef enum {
  ncclSuccess = 0,
  ncclUnhandledCudaError = 1,
  ncclSystemError = 2,
  ncclInternalError = 3,
  ncclInvalidArgument = 4,
  ncclInvalidUsage = 5,
  ncclRemoteError = 6,
  ncclInProgress = 7
} ncclResult_t;

typedef struct ncclComm* ncclComm_t;

typedef enum {
  ncclInt8 = 0,
  ncclUint8 = 1,
  ncclInt32 = 2,
  ncclUint32 = 3,
  ncclInt64 = 4,
  ncclUint64 = 5,
  ncclFloat16 = 6,
  ncclFloat = 7,
  ncclDouble = 8,
  ncclBfloat16 = 9
} ncclDataType_t;

typedef enum { ncclSum = 0, ncclProd = 1, ncclMax = 2, ncclMin = 3, ncclAvg = 4 } ncclRedOp_t;

/* ------------------------------------------- reference-compatible calls */

const char* ncclGetErrorString(ncclResult_t result);

/* rank >= 0: manual rank; `ip` is rank 0's address (NULL means 127.0.0.1).
 * rank == -1: Hera auto-bootstrap; `ip` is the Hera master's address, the
 * master assigns rank and world size (the caller's nRanks is ignored). */
ncclResult_t ncclCommInitRank(ncclComm_t* comm, int nRanks, int rank, const char* ip);
ncclResult_t ncclCommDestroy(ncclComm_t comm);
ncclResult_t ncclCommUserRank(const ncclComm_t comm, int* rank);
ncclResult_t ncclCommCount(const ncclComm_t comm, int* count);

/* In-place (sendbuff == recvbuff) and out-of-place are both valid.  Buffers
 * may be device memory, pinned host memory, or (on the CPU-only network path)
 * plain host memory.  All ten data types and all five operators work. */
ncclResult_t ncclAllReduce(const void* sendbuff, void* recvbuff, size_t count,
                           ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm,
                           cudaStream_t stream);

/* ---------------------------------------------------- additive extensions */

const char* mncclGetErrorString(ncclResult_t result);
ncclResult_t mncclCommInitRank(ncclComm_t* comm, int nRanks, int rank, const char* ip);
ncclResult_t mncclCommDestroy(ncclComm_t comm);
ncclResult_t mncclCommUserRank(const ncclComm_t comm, int* rank);
ncclResult_t mncclCommCount(const ncclComm_t comm, int* count);
ncclResult_t mncclAllReduce(const void* sendbuff, void* recvbuff, size_t count,
                            ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm,
                            cudaStream_t stream);

/* Algorithm ids accepted by mncclAllReduceEx / MINI_NCCL_ALGO. */
typedef enum {
  mncclAlgoAuto = 0,
  mncclAlgoLL = 1,        /* one-shot push, flag packed with data          */
  mncclAlgoOneShot = 2,   /* one-shot push + per-block barrier             */
  mncclAlgoTwoShot = 3,   /* P2P reduce-scatter (pull) + all-gather (push) */
  mncclAlgoNvls = 4,      /* multimem.ld_reduce + multimem.st              */
  mncclAlgoRing = 5,      /* host-driven ring over the one-sided transport */
  mncclAlgoLocal = 6,     /* one rank: copy with scale / conversion (reported only) */
  mncclAlgoPipe = 7       /* ordinary buffers: copy-in, reduce, copy-out blocks of one kernel, chunk by chunk */
} mncclAlgo_t;

/* AllReduce fused with a dtype conversion and a scale:
 *   recv[i] = (recv_type) ( scale * reduce_over_ranks( (wire_type) send[i] ) )
 * accumulation is fp32 in fixed rank order.  Supported triples
 * (send, wire, recv): any homogeneous triple, (f32,bf16,f32), (f32,bf16,bf16),
 * (bf16,bf16,f32).  algo = mncclAlgoAuto picks from the size table. */
ncclResult_t mncclAllReduceEx(const void* sendbuff, ncclDataType_t send_type, void* recvbuff,
                              ncclDataType_t recv_type, ncclDataType_t wire_type, size_t count,
                              ncclRedOp_t op, double scale, mncclAlgo_t algo, ncclComm_t comm,
                              cudaStream_t stream);

/* ReduceScatter / AllGather over the same data plane (building blocks of the
 * two-shot AllReduce and of the fused tensor-parallel kernels).
 * recvcount / sendcount are per-rank element counts. */
ncclResult_t mncclReduceScatter(const void* sendbuff, void* recvbuff, size_t recvcount,
                                ncclDataType_t datatype, ncclRedOp_t op, ncclComm_t comm,
                                cudaStream_t stream);
ncclResult_t mncclAllGather(const void* sendbuff, void* recvbuff, size_t sendcount,
                            ncclDataType_t datatype, ncclComm_t comm, cudaStream_t stream);

/* Symmetric allocations: collective calls (every rank, same order, same size).
 * Buffers obtained here are mapped into every peer (and bound to the NVSwitch
 * multicast object when NVLS is available), so collectives on them are
 * zero-copy.  Freed by mncclMemFree (collective) or at communicator destroy. */
ncclResult_t mncclMemAlloc(ncclComm_t comm, size_t bytes, void** ptr);
ncclResult_t mncclMemFree(ncclComm_t comm, void* ptr);

/* Peer views of a symmetric allocation (for fused compute+collective kernels).
 * peer_ptrs must hold nRanks entries; mc_ptr receives NULL when NVLS is off. */
ncclResult_t mncclMemPeerPointers(ncclComm_t comm, void* ptr, void** peer_ptrs, void** mc_ptr);

/* Registration of ordinary device buffers (cudaMalloc family): a collective call that exchanges
 * CUDA IPC handles once and keeps the opened mappings in a handle cache, after which the
 * peer-to-peer algorithms use the buffer in place (no staging).  NVLS needs memory from
 * mncclMemAlloc.  Every rank registers a buffer of the same size in the same call.
 * A registered buffer must be deregistered BEFORE it is freed: the registration is keyed by address,
 * and a later allocation in the same range would be reduced through the peers' mappings of the old
 * memory.  The library notices the change of allocation and refuses such a call (ncclInvalidUsage). */
ncclResult_t mncclCommRegister(ncclComm_t comm, void* buff, size_t bytes);
ncclResult_t mncclCommDeregister(ncclComm_t comm, void* buff);

/* Host barrier through the bootstrap store (not stream ordered). */
ncclResult_t mncclBarrier(ncclComm_t comm);

/* Failure handling.  mncclCommAbort sets the abort word seen by every kernel
 * of every local rank; waits then return within microseconds and the calls
 * report ncclInternalError.  mncclCommGetAsyncError never blocks. */
ncclResult_t mncclCommAbort(ncclComm_t comm);
ncclResult_t mncclCommGetAsyncError(ncclComm_t comm, ncclResult_t* async_error);

/* Observability: counters as one JSON object written into buf (NUL-terminated,
 * truncated to len). */
ncclResult_t mncclCommStats(ncclComm_t comm, char* buf, size_t len);

/* Which algorithm AllReduce would choose for this size (no launch). */
ncclResult_t mncclCommQueryAlgo(ncclComm_t comm, size_t bytes, ncclDataType_t datatype,
                                ncclRedOp_t op, int registered, mncclAlgo_t* algo);

/* Device-side descriptor of the communicator for user kernels that fuse a
 * collective (see csrc/kernels/comm_dev.h for the layout).  Copies at most
 * `len` bytes; returns the full size in *needed. */
ncclResult_t mncclCommDeviceHandle(ncclComm_t comm, void* out, size_t len, size_t* needed);

/* Launch tuning for the calls that follow (0 keeps the built-in value).  Every
 * rank must use the same values.  Meant for benchmarking sweeps. */
ncclResult_t mncclCommSetTuning(ncclComm_t comm, int max_blocks, int unroll);

/* One launch-tuning knob by the name of its environment variable without the MINI_NCCL_ prefix
 * ("LL_MAX_BYTES", "ONESHOT_MAX_BYTES", "NVLS_MIN_BYTES", "PIPE_MIN_BYTES", "PIPE_CHUNK_BYTES",
 * "MAX_BLOCKS", ...), for the calls that follow.  Every rank must use the same value.  The same knobs can be given per rank count in a table that
 * MINI_NCCL_TUNING_FILE names (lines "<nranks> <KNOB> <value>", written by benchmarks/tune.py);
 * environment variables win over the table. */
ncclResult_t mncclCommSetKnob(ncclComm_t comm, const char* name, long long value);

unsigned mncclVersion(void);

#ifdef __cplusplus
}
#endif

#endif /* MINI_NCCL_B200_API_H_ */
