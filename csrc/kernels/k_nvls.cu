// Kernel instantiations: NVLS AllReduce (multimem.ld_reduce + multimem.st).
#include "kernels/dispatch.cuh"

namespace mnccl {
namespace dev {

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) nvls_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, true, kAllReduce, 4>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) nvls_kernel_u8(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, true, kAllReduce, 8>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
struct NvlsF {
  static cudaError_t go(const LaunchCtx& x) {
    if (x.vranks > 1 || x.occupancy_out) return kNoKernel;  // multimem needs a real multicast mapping
    if (x.spec->unroll == 8) return fire(nvls_kernel_u8<InT, WireT, OutT, OP>, nvls_kernel_u8<InT, WireT, OutT, OP>, x);
    return fire(nvls_kernel<InT, WireT, OutT, OP>, nvls_kernel<InT, WireT, OutT, OP>, x);
  }
};
cudaError_t dispatch_nvls_ar(const LaunchCtx& x) { return dispatch_nvls<NvlsF>(x); }

}  // namespace dev
}  // namespace mnccl
