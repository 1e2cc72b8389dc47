// Type / operator dispatch shared by the kernel translation units.
#pragma once
#include <cuda_runtime.h>

#include "kernels/coll_kernels.cuh"
#include "kernels/launch.h"

namespace mnccl {
namespace dev {

struct LaunchCtx {
  const LaunchSpec* spec;
  const KParams* p;      // normal launch
  const KParams* table;  // emulated launch
  int vranks;            // 0: query only (does the kernel exist?), 1: normal, >1: emulated
  cudaStream_t stream;
  int* occupancy_out;    // non-null: report max co-resident blocks per SM instead of launching
};

template <typename KernelT, typename EmuT>
inline cudaError_t fire(KernelT k, EmuT ke, const LaunchCtx& x) {
  if (x.vranks == 0) return cudaSuccess;
  const int threads = x.spec->nthreads;
  if (x.occupancy_out) {
    return cudaOccupancyMaxActiveBlocksPerMultiprocessor(x.occupancy_out, ke, threads, 0);
  }
  if (x.vranks == 1) {
    k<<<x.spec->nblocks, threads, 0, x.stream>>>(*x.p);
    return cudaGetLastError();
  }
  const KParams* table = x.table;
  int nblk = x.spec->nblocks;
  void* args[] = {const_cast<KParams**>(&table), &nblk};
  return cudaLaunchCooperativeKernel(reinterpret_cast<void*>(ke), dim3(nblk * x.vranks), dim3(threads), args, 0,
                                     x.stream);
}

constexpr cudaError_t kNoKernel = cudaErrorInvalidDeviceFunction;

inline bool homogeneous(const LaunchSpec& s) { return s.in == s.wire && s.in == s.out; }
inline int op_index(RedOp op) { return op == RedOp::Avg ? 0 : static_cast<int>(op); }

// Calls F<In, Wire, Out, OP>::go(ctx) for the spec's types and operator.
// Homogeneous triples support every operator, mixed triples Sum / Avg only.
#define MNCCL_DISPATCH_OPS(F, T, ctx, op)                                   \
  switch (op) {                                                             \
    case 0: return F<T, T, T, 0>::go(ctx);                                  \
    case 1: return F<T, T, T, 1>::go(ctx);                                  \
    case 2: return F<T, T, T, 2>::go(ctx);                                  \
    case 3: return F<T, T, T, 3>::go(ctx);                                  \
  }                                                                         \
  return kNoKernel;

template <template <typename, typename, typename, int> class F>
inline cudaError_t dispatch_all(const LaunchCtx& ctx) {
  const LaunchSpec& s = *ctx.spec;
  const int op = op_index(s.op);
  if (homogeneous(s)) {
    switch (s.in) {
      case DType::Int8: MNCCL_DISPATCH_OPS(F, int8_t, ctx, op)
      case DType::Uint8: MNCCL_DISPATCH_OPS(F, uint8_t, ctx, op)
      case DType::Int32: MNCCL_DISPATCH_OPS(F, int32_t, ctx, op)
      case DType::Uint32: MNCCL_DISPATCH_OPS(F, uint32_t, ctx, op)
      case DType::Int64: MNCCL_DISPATCH_OPS(F, int64_t, ctx, op)
      case DType::Uint64: MNCCL_DISPATCH_OPS(F, uint64_t, ctx, op)
      case DType::Float16: MNCCL_DISPATCH_OPS(F, __half, ctx, op)
      case DType::Float32: MNCCL_DISPATCH_OPS(F, float, ctx, op)
      case DType::Float64: MNCCL_DISPATCH_OPS(F, double, ctx, op)
      case DType::Bfloat16: MNCCL_DISPATCH_OPS(F, __nv_bfloat16, ctx, op)
    }
    return kNoKernel;
  }
  if (op != 0) return kNoKernel;
  if (s.in == DType::Float32 && s.wire == DType::Bfloat16 && s.out == DType::Float32)
    return F<float, __nv_bfloat16, float, 0>::go(ctx);
  if (s.in == DType::Float32 && s.wire == DType::Bfloat16 && s.out == DType::Bfloat16)
    return F<float, __nv_bfloat16, __nv_bfloat16, 0>::go(ctx);
  if (s.in == DType::Bfloat16 && s.wire == DType::Bfloat16 && s.out == DType::Float32)
    return F<__nv_bfloat16, __nv_bfloat16, float, 0>::go(ctx);
  return kNoKernel;
}

// Sum-only dispatch over the types the switch can reduce (NVLS).
template <template <typename, typename, typename, int> class F>
inline cudaError_t dispatch_nvls(const LaunchCtx& ctx) {
  const LaunchSpec& s = *ctx.spec;
  if (op_index(s.op) != 0) return kNoKernel;
  if (homogeneous(s)) {
    switch (s.in) {
      case DType::Float16: return F<__half, __half, __half, 0>::go(ctx);
      case DType::Float32: return F<float, float, float, 0>::go(ctx);
      case DType::Bfloat16: return F<__nv_bfloat16, __nv_bfloat16, __nv_bfloat16, 0>::go(ctx);
      default: return kNoKernel;
    }
  }
  if (s.in == DType::Float32 && s.wire == DType::Bfloat16 && s.out == DType::Float32)
    return F<float, __nv_bfloat16, float, 0>::go(ctx);
  if (s.in == DType::Float32 && s.wire == DType::Bfloat16 && s.out == DType::Bfloat16)
    return F<float, __nv_bfloat16, __nv_bfloat16, 0>::go(ctx);
  if (s.in == DType::Bfloat16 && s.wire == DType::Bfloat16 && s.out == DType::Float32)
    return F<__nv_bfloat16, __nv_bfloat16, float, 0>::go(ctx);
  return kNoKernel;
}

// Copy-only dispatch by element size (AllGather).
template <template <typename, typename, typename, int> class F>
inline cudaError_t dispatch_bytes(const LaunchCtx& ctx) {
  const LaunchSpec& s = *ctx.spec;
  if (!homogeneous(s)) return kNoKernel;
  switch (dtype_size(s.in)) {
    case 1: return F<uint8_t, uint8_t, uint8_t, 0>::go(ctx);
    case 2: return F<uint16_t, uint16_t, uint16_t, 0>::go(ctx);
    case 4: return F<uint32_t, uint32_t, uint32_t, 0>::go(ctx);
    case 8: return F<uint64_t, uint64_t, uint64_t, 0>::go(ctx);
  }
  return kNoKernel;
}

}  // namespace dev
}  // namespace mnccl
