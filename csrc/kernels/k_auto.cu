// Kernel instantiations: the peer-to-peer two-shot AllReduce on ordinary device buffers with lazy
// direct access (one type in, on the wire and out; every operator).
#include "kernels/dispatch.cuh"

namespace mnccl {
namespace dev {

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) twoshot_auto_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  twoshot_auto_body<InT, OP>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) twoshot_auto_kernel_emu(const KParams* table, int nblk) {
  __shared__ BlockCtl ctl;
  twoshot_auto_body<InT, OP>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
struct TwoShotAutoF {
  static cudaError_t go(const LaunchCtx& x) {
    return fire(twoshot_auto_kernel<InT, WireT, OutT, OP>, twoshot_auto_kernel_emu<InT, WireT, OutT, OP>, x);
  }
};
cudaError_t dispatch_twoshot_auto(const LaunchCtx& x) {
  if (!homogeneous(*x.spec)) return kNoKernel;
  return dispatch_all<TwoShotAutoF>(x);
}

}  // namespace dev
}  // namespace mnccl
