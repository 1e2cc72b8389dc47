// Host-side launch interface of the collective kernels.
#pragma once
#include <cuda_runtime.h>

#include "core/dtype.h"
#include "kernels/comm_dev.h"

namespace mnccl {

enum class Algo : int { Auto = 0, LL = 1, OneShot = 2, TwoShot = 3, Nvls = 4, Ring = 5, Local = 6, Pipe = 7, HostSync = 8 };
enum class Mode : int { AllReduce = 0, ReduceScatter = 1, AllGather = 2 };

inline const char* algo_name(Algo a) {
  switch (a) {
    case Algo::Auto: return "auto"; case Algo::LL: return "ll"; case Algo::OneShot: return "oneshot";
    case Algo::TwoShot: return "twoshot"; case Algo::Nvls: return "nvls"; case Algo::Ring: return "ring";
    case Algo::Local: return "local"; case Algo::Pipe: return "pipe"; case Algo::HostSync: return "hostsync";
  }
  return "?";
}

struct LaunchSpec {
  Algo algo = Algo::OneShot;
  Mode mode = Mode::AllReduce;
  DType in = DType::Float32, wire = DType::Float32, out = DType::Float32;
  RedOp op = RedOp::Sum;  // Avg is launched as Sum; the factor travels in CollArgs
  int nblocks = 1;
  int nthreads = 512;
  int unroll = 4;  // vectors in flight per thread in the NVLS kernels (4 or 8)
  bool pipe_nvls = false;  // Algo::Pipe: reduce through the switch (multimem) instead of peer loads / stores
  bool auto_direct = false;  // Algo::TwoShot on ordinary buffers: the kernel that goes direct once every rank has mapped every buffer
};

// True when a kernel exists for this combination of algorithm, mode, types
// and operator.
bool kernel_exists(const LaunchSpec& spec);

// Launch on one rank (the normal case).  `p` is passed by value to the kernel.
cudaError_t launch_collective(const LaunchSpec& spec, const KParams& p, cudaStream_t stream);

// Single-GPU emulation of `vranks` ranks: ONE cooperative launch whose grid is
// vranks * spec.nblocks blocks; block g acts as block g % nblocks of rank
// g / nblocks and reads its parameters from table[g / nblocks] (device
// memory).  All virtual ranks' buffers live on the current device.  Used by
// tests and debugging; the blocks of different virtual ranks wait on one
// another, which is only safe because a cooperative launch makes them
// co-resident.
cudaError_t launch_collective_emulated(const LaunchSpec& spec, const KParams* table, int vranks,
                                       cudaStream_t stream);

// Largest grid per virtual rank that a cooperative launch of this kernel can
// hold on the current device.
int max_emulated_blocks(const LaunchSpec& spec, int vranks);

}  // namespace mnccl
