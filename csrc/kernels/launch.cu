#include "kernels/launch.h"

#include "kernels/dispatch.cuh"

namespace mnccl {
namespace dev {
cudaError_t dispatch_local(const LaunchCtx&);
cudaError_t dispatch_ll(const LaunchCtx&);
cudaError_t dispatch_oneshot(const LaunchCtx&);
cudaError_t dispatch_twoshot_ar(const LaunchCtx&);
cudaError_t dispatch_twoshot_auto(const LaunchCtx&);
cudaError_t dispatch_nvls_ar(const LaunchCtx&);
cudaError_t dispatch_rs(const LaunchCtx&);
cudaError_t dispatch_rs_nvls(const LaunchCtx&);
cudaError_t dispatch_ag(const LaunchCtx&);
cudaError_t dispatch_pipe(const LaunchCtx&);
cudaError_t dispatch_gather_reduce(const LaunchCtx&);
cudaError_t dispatch_pipe_nvls(const LaunchCtx&);
}  // namespace dev

namespace {
cudaError_t route(const dev::LaunchCtx& x) {
  const LaunchSpec& s = *x.spec;
  switch (s.mode) {
    case Mode::AllReduce:
      switch (s.algo) {
        case Algo::Local: return dev::dispatch_local(x);
        case Algo::LL: return dev::dispatch_ll(x);
        case Algo::OneShot: return dev::dispatch_oneshot(x);
        case Algo::TwoShot: return s.auto_direct ? dev::dispatch_twoshot_auto(x) : dev::dispatch_twoshot_ar(x);
        case Algo::Nvls: return dev::dispatch_nvls_ar(x);
        case Algo::Pipe: return s.pipe_nvls ? dev::dispatch_pipe_nvls(x) : dev::dispatch_pipe(x);
        case Algo::HostSync: return dev::dispatch_gather_reduce(x);
        default: return dev::kNoKernel;
      }
    case Mode::ReduceScatter:
      if (s.algo == Algo::TwoShot) return dev::dispatch_rs(x);
      if (s.algo == Algo::Nvls) return dev::dispatch_rs_nvls(x);
      return dev::kNoKernel;
    case Mode::AllGather:
      if (s.algo == Algo::TwoShot) return dev::dispatch_ag(x);
      return dev::kNoKernel;
  }
  return dev::kNoKernel;
}
}  // namespace

bool kernel_exists(const LaunchSpec& spec) {
  dev::LaunchCtx x{&spec, nullptr, nullptr, 0, nullptr, nullptr};
  return route(x) == cudaSuccess;
}

cudaError_t launch_collective(const LaunchSpec& spec, const KParams& p, cudaStream_t stream) {
  // Only kernels with per-block barrier state are bound by kMaxBlocks.
  const int max_blocks = (spec.algo == Algo::Local || spec.algo == Algo::HostSync) ? 65535 : kMaxBlocks;
  if (spec.nblocks < 1 || spec.nblocks > max_blocks || spec.nthreads < 32 || spec.nthreads > 512)
    return cudaErrorInvalidConfiguration;
  if (spec.auto_direct && spec.nblocks > kAutoBlocks) return cudaErrorInvalidConfiguration;
  dev::LaunchCtx x{&spec, &p, nullptr, 1, stream, nullptr};
  return route(x);
}

cudaError_t launch_collective_emulated(const LaunchSpec& spec, const KParams* table, int vranks,
                                       cudaStream_t stream) {
  if (vranks < 2 || vranks > kMaxRanks || spec.nblocks < 1 || spec.nblocks > kMaxBlocks || spec.nthreads < 32 ||
      spec.nthreads > 512)
    return cudaErrorInvalidConfiguration;
  if (spec.nblocks > max_emulated_blocks(spec, vranks)) return cudaErrorCooperativeLaunchTooLarge;
  dev::LaunchCtx x{&spec, nullptr, table, vranks, stream, nullptr};
  return route(x);
}

int max_emulated_blocks(const LaunchSpec& spec, int vranks) {
  int per_sm = 0;
  dev::LaunchCtx x{&spec, nullptr, nullptr, 2, nullptr, &per_sm};
  if (route(x) != cudaSuccess || per_sm <= 0) return 0;
  int dev_id = 0, sms = 0;
  if (cudaGetDevice(&dev_id) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev_id) != cudaSuccess) return 0;
  int total = per_sm * sms;
  int per_rank = total / (vranks > 0 ? vranks : 1);
  return per_rank > kMaxBlocks ? kMaxBlocks : per_rank;
}

}  // namespace mnccl
