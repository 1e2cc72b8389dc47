// Kernel instantiations: the pipelined AllReduce for buffers outside symmetric memory
// (copy-in, reduce and copy-out blocks of one kernel working chunk by chunk; see pipe_body).
#include "kernels/dispatch.cuh"

namespace mnccl {
namespace dev {

// (The peer-to-peer form spills 100 to 400 bytes per thread under the 128-register cap of 512-thread
// blocks; 256-thread blocks are spill-free but measured slower still on two GPUs, 1200 against 800 us for
// 256 MiB, so the larger blocks stay.  This form is only taken when asked for: algo = pipe.)
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) pipe_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  pipe_body<InT, WireT, OutT, OP, false>(P, blockIdx.x, gridDim.x, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) pipe_kernel_emu(const KParams* table, int nblk) {
  __shared__ BlockCtl ctl;
  pipe_body<InT, WireT, OutT, OP, false>(table[blockIdx.x / nblk], blockIdx.x % nblk, nblk, ctl);
}
template <typename InT, typename WireT, typename OutT, int OP>
__global__ void __launch_bounds__(512) pipe_nvls_kernel(const __grid_constant__ KParams P) {
  __shared__ BlockCtl ctl;
  pipe_body<InT, WireT, OutT, OP, true>(P, blockIdx.x, gridDim.x, ctl);
}

template <typename InT, typename WireT, typename OutT, int OP>
struct PipeF {
  static cudaError_t go(const LaunchCtx& x) {
    return fire(pipe_kernel<InT, WireT, OutT, OP>, pipe_kernel_emu<InT, WireT, OutT, OP>, x);
  }
};
template <typename InT, typename WireT, typename OutT, int OP>
struct PipeNvlsF {
  static cudaError_t go(const LaunchCtx& x) {
    if (x.vranks > 1 || x.occupancy_out) return kNoKernel;  // multimem needs a real multicast mapping
    return fire(pipe_nvls_kernel<InT, WireT, OutT, OP>, pipe_nvls_kernel<InT, WireT, OutT, OP>, x);
  }
};

cudaError_t dispatch_pipe(const LaunchCtx& x) { return dispatch_all<PipeF>(x); }
cudaError_t dispatch_pipe_nvls(const LaunchCtx& x) { return dispatch_nvls<PipeNvlsF>(x); }

}  // namespace dev
}  // namespace mnccl
