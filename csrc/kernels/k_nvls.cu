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
// Two messages in one launch: blocks [0, nb_first) reduce the first through the switch, the others
// the second with peer loads and stores in rank order.  The switch's reduction rate, not the links,
// bounds the NVLS path (a handful of blocks saturates it and the links stay ~40 % idle), so a slice
// of a large message can travel peer-to-peer at the same time.
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) nvls_split_kernel(const __grid_constant__ KParamsSplit P) {
  __shared__ BlockCtl ctl;
  const int blk = blockIdx.x, nblk = gridDim.x;
  block_begin(P.comm, blk, ctl);
  if (blk < P.nb_first) twoshot_core<InT, WireT, OutT, OP, true, kAllReduce, 4>(P.comm, P.args, blk, blk, P.nb_first, ctl);
  else twoshot_core<InT, WireT, OutT, OP, false, kAllReduce, 4>(P.comm, P.args2, blk, blk - P.nb_first, nblk - P.nb_first, ctl);
  block_end(P.comm, blk, nblk, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
struct NvlsSplitF {
  static cudaError_t go(const LaunchCtx& x) {
    if (x.vranks == 0) return cudaSuccess;
    if (x.vranks > 1 || x.occupancy_out || x.split == nullptr) return kNoKernel;
    nvls_split_kernel<InT, WireT, OutT, OP><<<x.spec->nblocks, x.spec->nthreads, 0, x.stream>>>(*x.split);
    return cudaGetLastError();
  }
};
cudaError_t dispatch_nvls_split(const LaunchCtx& x) { return dispatch_nvls<NvlsSplitF>(x); }

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
