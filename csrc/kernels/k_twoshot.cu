// Kernel instantiations: two-shot P2P AllReduce (all types and operators).
#include "kernels/dispatch.cuh"

namespace mnccl {
namespace dev {

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) twoshot_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, false, kAllReduce>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) twoshot_kernel_emu(const KParams* table, int nblk) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, false, kAllReduce>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
struct TwoShotF {
  static cudaError_t go(const LaunchCtx& x) {
    return fire(twoshot_kernel<InT, WireT, OutT, OP>, twoshot_kernel_emu<InT, WireT, OutT, OP>, x);
  }
};
cudaError_t dispatch_twoshot_ar(const LaunchCtx& x) { return dispatch_all<TwoShotF>(x); }

}  // namespace dev
}  // namespace mnccl
