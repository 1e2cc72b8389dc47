// Kernel instantiations: ReduceScatter and AllGather (P2P and NVLS).
#include "kernels/dispatch.cuh"

namespace mnccl {
namespace dev {

template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) rs_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, false, kReduceScatter>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) rs_kernel_emu(const KParams* table, int nblk) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, false, kReduceScatter>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) rs_nvls_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, true, kReduceScatter>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) ag_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, false, kAllGather>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) ag_kernel_emu(const KParams* table, int nblk) {
  __shared__ BlockCtl ctl;
  twoshot_body<InT, WireT, OutT, OP, false, kAllGather>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}

template <typename InT, typename WireT, typename OutT, int OP>
struct RsF {
  static cudaError_t go(const LaunchCtx& x) {
    return fire(rs_kernel<InT, WireT, OutT, OP>, rs_kernel_emu<InT, WireT, OutT, OP>, x);
  }
};
template <typename InT, typename WireT, typename OutT, int OP>
struct RsNvlsF {
  static cudaError_t go(const LaunchCtx& x) {
    if (x.vranks > 1 || x.occupancy_out) return kNoKernel;  // multimem needs a real multicast mapping
    return fire(rs_nvls_kernel<InT, WireT, OutT, OP>, rs_nvls_kernel<InT, WireT, OutT, OP>, x);
  }
};
template <typename InT, typename WireT, typename OutT, int OP>
struct AgF {
  static cudaError_t go(const LaunchCtx& x) {
    return fire(ag_kernel<InT, WireT, OutT, OP>, ag_kernel_emu<InT, WireT, OutT, OP>, x);
  }
};

cudaError_t dispatch_rs(const LaunchCtx& x) {
  if (!homogeneous(*x.spec)) return kNoKernel;
  return dispatch_all<RsF>(x);
}
cudaError_t dispatch_rs_nvls(const LaunchCtx& x) {
  if (!homogeneous(*x.spec)) return kNoKernel;
  return dispatch_nvls<RsNvlsF>(x);
}
cudaError_t dispatch_ag(const LaunchCtx& x) { return dispatch_bytes<AgF>(x); }

}  // namespace dev
}  // namespace mnccl
