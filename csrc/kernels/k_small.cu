// Kernel instantiations: N == 1 local copy, LL and one-shot AllReduce.
#include "kernels/dispatch.cuh"

namespace mnccl {
namespace dev {

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) local_kernel(const __grid_constant__ KParams P) {
  local_body<InT, OutT>(P, blockIdx.x, gridDim.x);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) local_kernel_emu(const KParams* table, int nblk) {
  local_body<InT, OutT>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk);
}

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) ll_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  ll_body<InT, WireT, OutT, OP>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) ll_kernel_emu(const KParams* table, int nblk) {
  __shared__ BlockCtl ctl;
  ll_body<InT, WireT, OutT, OP>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) oneshot_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  oneshot_body<InT, WireT, OutT, OP>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) oneshot_kernel_emu(const KParams* table, int nblk) {
  __shared__ BlockCtl ctl;
  oneshot_body<InT, WireT, OutT, OP>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) gather_reduce_kernel(const __grid_constant__ KParams P) {
  gather_reduce_body<InT, WireT, OutT, OP>(P, blockIdx.x, gridDim.x);
}
template <typename InT, typename WireT, typename OutT, int OP>
struct GatherReduceF {
  static cudaError_t go(const LaunchCtx& x) {
    if (x.vranks > 1 || x.occupancy_out) return kNoKernel;  // one rank per launch by construction
    return fire(gather_reduce_kernel<InT, WireT, OutT, OP>, gather_reduce_kernel<InT, WireT, OutT, OP>, x);
  }
};

template <typename InT, typename WireT, typename OutT, int OP>
struct LocalF {
  static cudaError_t go(const LaunchCtx& x) {
    if (OP != 0) return kNoKernel;
    return fire(local_kernel<InT, WireT, OutT, 0>, local_kernel_emu<InT, WireT, OutT, 0>, x);
  }
};
template <typename InT, typename WireT, typename OutT, int OP>
struct LLF {
  static cudaError_t go(const LaunchCtx& x) {
    return fire(ll_kernel<InT, WireT, OutT, OP>, ll_kernel_emu<InT, WireT, OutT, OP>, x);
  }
};
template <typename InT, typename WireT, typename OutT, int OP>
struct OneShotF {
  static cudaError_t go(const LaunchCtx& x) {
    return fire(oneshot_kernel<InT, WireT, OutT, OP>, oneshot_kernel_emu<InT, WireT, OutT, OP>, x);
  }
};

cudaError_t dispatch_local(const LaunchCtx& x) {
  // A single rank reduces nothing: every operator is the identity (plus scale).
  LaunchSpec s = *x.spec;
  s.op = RedOp::Sum;
  LaunchCtx y = x;
  y.spec = &s;
  return dispatch_all<LocalF>(y);
}
cudaError_t dispatch_gather_reduce(const LaunchCtx& x) { return dispatch_all<GatherReduceF>(x); }
cudaError_t dispatch_ll(const LaunchCtx& x) { return dispatch_all<LLF>(x); }
cudaError_t dispatch_oneshot(const LaunchCtx& x) { return dispatch_all<OneShotF>(x); }

}  // namespace dev
}  // namespace mnccl
