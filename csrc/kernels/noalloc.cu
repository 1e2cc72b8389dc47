// See noalloc.h: an AllReduce over several buffers of one GPU that allocates
// nothing.  Scratch (control words + inboxes of every virtual rank) is a static
// device array; parameters go by value; the launch is cooperative because the
// virtual ranks' blocks wait on one another.
#include "kernels/noalloc.h"

#include <cuda_runtime.h>

#include <cstddef>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "core/dtype.h"
#include "kernels/coll_kernels.cuh"

namespace mnccl {
namespace {

constexpr size_t align_up_c(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Layout of one virtual rank's control segment inside the static array.
constexpr size_t kSigBytes = align_up_c(sizeof(uint32_t) * kMaxBlocks * kMaxRanks, 4096);
constexpr size_t kLocalBytes = align_up_c(sizeof(LocalState), 4096);
constexpr size_t kClearBytes = kSigBytes + kLocalBytes;  // cleared at the start of every call
constexpr size_t kInboxSlot = kNoAllocMaxBytes;
constexpr size_t kInboxBytes = 2 * size_t(kNoAllocMaxRanks) * kInboxSlot;
constexpr size_t kCtrlBytes = kClearBytes + kInboxBytes;
constexpr size_t kScratchBytes = size_t(kNoAllocMaxRanks) * kCtrlBytes;

// The scratch itself.  In host code this name is only a handle for the runtime
// (cudaGetSymbolAddress); device code could name it directly.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kScratchBytes];

struct NoAllocParams {
  KParams rank[kNoAllocMaxRanks];
};
static_assert(sizeof(NoAllocParams) <= 4000, "kernel parameters must fit the 4 KB parameter space");

template <typename T, int OP>
__global__ void __launch_bounds__(512) noalloc_oneshot_kernel(const __grid_constant__ NoAllocParams P, int nblk) {
  __shared__ dev::BlockCtl ctl;
  dev::oneshot_body<T, T, T, OP>(P.rank[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}

template <typename T>
cudaError_t launch_typed(int op, const NoAllocParams& p, int nranks, int nblk, int threads, cudaStream_t stream) {
  void* args[] = {const_cast<NoAllocParams*>(&p), &nblk};
  const void* fn = nullptr;
  switch (op) {
    case 0: fn = reinterpret_cast<const void*>(noalloc_oneshot_kernel<T, 0>); break;
    case 1: fn = reinterpret_cast<const void*>(noalloc_oneshot_kernel<T, 1>); break;
    case 2: fn = reinterpret_cast<const void*>(noalloc_oneshot_kernel<T, 2>); break;
    case 3: fn = reinterpret_cast<const void*>(noalloc_oneshot_kernel<T, 3>); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaLaunchCooperativeKernel(fn, dim3(nblk * nranks), dim3(threads), args, 0, stream);
}

// Per-device address of the scratch array, looked up once with that device current.
std::mutex g_mu;
unsigned char* g_scratch_addr[64] = {nullptr};

cudaError_t scratch_for_current_device(unsigned char** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  std::lock_guard<std::mutex> lk(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess) return e;
    g_scratch_addr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_addr[dev];
  return cudaSuccess;
}

}  // namespace

// Fills the control part (barrier words, per-rank state) of every virtual rank's scratch with `byte`, as
// a call that was cut short might leave it; the next call must not care.  Not exported: reached through
// the test-suite's own library only (csrc/testing/hooks.cc).
int noalloc_dirty_control(int byte) {
  unsigned char* scratch = nullptr;
  if (scratch_for_current_device(&scratch) != cudaSuccess) return 1;
  for (int r = 0; r < kNoAllocMaxRanks; ++r)
    if (cudaMemset(scratch + size_t(r) * kCtrlBytes, byte, kClearBytes) != cudaSuccess) return 2;
  return cudaDeviceSynchronize() == cudaSuccess ? 0 : 3;
}

}  // namespace mnccl

using namespace mnccl;

extern "C" {
#define MNCCL_EXPORT __attribute__((visibility("default")))

MNCCL_EXPORT size_t mncclNoAllocScratchBytes(void) { return kScratchBytes; }

// What the last call on the current device left in the static scratch: 0 when every wait of its
// kernel completed, else the status of the first wait that gave up (1 = ran out of its two seconds,
// 2 = aborted) with, in *detail, (block << 16) | virtual rank waited for.  A kernel whose wait gave up
// returns early, so the output of that call is incomplete although the call itself returned
// ncclSuccess: callers that must know ask here.  Synchronises `stream` and copies eight bytes per
// virtual rank out of the scratch; allocates nothing.  The next call's clearing erases the record.
MNCCL_EXPORT ncclResult_t mncclNoAllocLastStatus(cudaStream_t stream, unsigned* status, unsigned* detail) {
  if (!status) return ncclInvalidArgument;
  unsigned char* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
  *status = 0;
  if (detail) *detail = 0;
  for (int r = 0; r < kNoAllocMaxRanks && e == cudaSuccess; ++r) {
    unsigned words[2] = {0, 0};
    e = cudaMemcpy(words, scratch + size_t(r) * kCtrlBytes + kSigBytes + offsetof(LocalState, status), sizeof(words),
                   cudaMemcpyDeviceToHost);
    if (e == cudaSuccess && words[0] != 0 && *status == 0) {
      *status = words[0];
      if (detail) *detail = words[1];
    }
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    return ncclUnhandledCudaError;
  }
  return ncclSuccess;
}

MNCCL_EXPORT ncclResult_t mncclLocalAllReduceNoAlloc(const void* const* send, void* const* recv, int nbuffers,
                                                     size_t count, ncclDataType_t datatype, ncclRedOp_t op,
                                                     cudaStream_t stream) {
  if (!send || !recv) return ncclInvalidArgument;
  if (nbuffers < 2 || nbuffers > kNoAllocMaxRanks) {
    fprintf(stderr, "[Mini-NCCL] mncclLocalAllReduceNoAlloc: %d buffers requested, supported: 2..%d\n", nbuffers,
            static_cast<int>(kNoAllocMaxRanks));
    return ncclInvalidArgument;
  }
  if (!valid_dtype(datatype) || !valid_op(op)) return ncclInvalidArgument;
  const DType t = static_cast<DType>(datatype);
  if (t != DType::Float32 && t != DType::Float16 && t != DType::Bfloat16 && t != DType::Int32) {
    fprintf(stderr, "[Mini-NCCL] mncclLocalAllReduceNoAlloc: type %s is not supported (fp32, fp16, bf16, int32 are)\n",
            dtype_name(t));
    return ncclInvalidArgument;
  }
  if (count == 0) return ncclSuccess;
  const size_t bytes = count * dtype_size(t);
  if (bytes > kNoAllocMaxBytes) {
    fprintf(stderr, "[Mini-NCCL] mncclLocalAllReduceNoAlloc: %zu bytes per buffer exceed the static scratch (max %d bytes)\n",
            bytes, static_cast<int>(kNoAllocMaxBytes));
    return ncclInvalidArgument;
  }
  for (int r = 0; r < nbuffers; ++r)
    if (!send[r] || !recv[r]) return ncclInvalidArgument;

  unsigned char* scratch = nullptr;
  cudaError_t e = scratch_for_current_device(&scratch);
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    fprintf(stderr, "[Mini-NCCL] mncclLocalAllReduceNoAlloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
    return ncclUnhandledCudaError;
  }
  // Start from clean barrier words and per-rank state, whatever the last call left.
  for (int r = 0; r < nbuffers; ++r) {
    e = cudaMemsetAsync(scratch + size_t(r) * kCtrlBytes, 0, kClearBytes, stream);
    if (e != cudaSuccess) {
      (void)cudaGetLastError();
      return ncclUnhandledCudaError;
    }
  }
  NoAllocParams p;
  memset(&p, 0, sizeof(p));
  const bool is_float = t != DType::Int32;
  const double factor = (op == ncclAvg) ? 1.0 / nbuffers : 1.0;
  for (int r = 0; r < nbuffers; ++r) {
    CommDev& c = p.rank[r].comm;
    c.rank = r;
    c.nranks = nbuffers;
    for (int q = 0; q < nbuffers; ++q) c.ctrl[q] = reinterpret_cast<char*>(scratch + size_t(q) * kCtrlBytes);
    c.spin_timeout_ns = 2000000000ull;
    c.off_sig = 0;
    c.off_local = kSigBytes;
    c.off_inbox = kClearBytes;
    c.inbox_slot_bytes = kInboxSlot;
    CollArgs& a = p.rank[r].args;
    a.send = send[r];
    a.recv = recv[r];
    a.count = count;
    a.scale_f = static_cast<float>(factor);
    a.scale_d = factor;
    a.int_div = (op == ncclAvg && !is_float) ? nbuffers : 0;
  }
  const size_t vecs = (bytes + 15) / 16;
  const int threads = vecs <= 256 ? 256 : 512;
  int nblk = static_cast<int>((vecs + threads - 1) / threads);
  if (nblk > 8) nblk = 8;  // 4 ranks x 8 blocks: co-resident on any GPU this library targets
  const int opi = (op == ncclAvg) ? 0 : static_cast<int>(op);
  switch (t) {
    case DType::Float32: e = launch_typed<float>(opi, p, nbuffers, nblk, threads, stream); break;
    case DType::Float16: e = launch_typed<__half>(opi, p, nbuffers, nblk, threads, stream); break;
    case DType::Bfloat16: e = launch_typed<__nv_bfloat16>(opi, p, nbuffers, nblk, threads, stream); break;
    default: e = launch_typed<int32_t>(opi, p, nbuffers, nblk, threads, stream); break;
  }
  if (e != cudaSuccess) {
    (void)cudaGetLastError();
    fprintf(stderr, "[Mini-NCCL] mncclLocalAllReduceNoAlloc: launch failed: %s\n", cudaGetErrorString(e));
    return ncclUnhandledCudaError;
  }
  return ncclSuccess;
}

}  // extern "C"
