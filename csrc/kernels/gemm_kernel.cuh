// The kernel template of the sm_100a bf16 GEMM and its launcher (see gemm_sm100.cu for
// the description of the roles).  Included by the translation units that instantiate it
// with an epilogue: gemm_sm100.cu (plain store) and gemm_fused.cu (reduce-scatter push,
// all-gather feed).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels/gemm_sm100.h"
#include "kernels/sm100_ptx.cuh"

namespace mnccl {
namespace gemm {

using namespace sm100;


__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Words of the per-device error buffer (error_word()): [0] first failed wait, [1] fused kernels
// started, [2] fused kernels finished (device-resident counters behind the watchdog's view).
__device__ __forceinline__ void st_volatile_sys_u32(volatile uint32_t* p, uint32_t v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// First CTA in: a fused kernel is in flight (what the communicator's watchdog times).
__device__ __forceinline__ void fused_kernel_started(const GemmArgs& g) {
  if (g.comm_progress == nullptr || g.err == nullptr || blockIdx.x != 0) return;
  const uint32_t s = atomicAdd(g.err + 1, 1u) + 1u;
  st_volatile_sys_u32(g.comm_progress + 4, s);
}

// A CTA's waits gave up with `code` (GemmAbort): device error word, and the communicator's status
// words, which make the watchdog set the abort word and the communicator fail for good.
__device__ __forceinline__ void report_failure(const GemmArgs& g, uint32_t code) {
  if (code == 0u || g.err == nullptr) return;
  if (atomicCAS(g.err, 0u, code) == 0u && g.comm_progress != nullptr) {
    st_volatile_sys_u32(g.comm_progress + 3, (static_cast<uint32_t>(blockIdx.x) << 16) | 0x8000u | code);
    __threadfence_system();
    st_volatile_sys_u32(g.comm_progress + 2, code == kGemmAborted ? 2u /*kDevAborted*/ : 1u /*kDevTimeout*/);
  }
}

// Last CTA out publishes the new epoch of a fused op (see GemmArgs::epoch_ptr).  Returns true in
// that CTA, whose caller then gives the epilogue its say (Epilogue::last_cta_out).
__device__ __forceinline__ bool finish_epoch(const GemmArgs& g, uint32_t epoch) {
  if (g.epoch_ptr == nullptr) return false;
  __threadfence();
  const uint32_t t = atomicAdd(g.ticket_ptr, 1u);
  if (t == gridDim.x - 1) {
    *g.ticket_ptr = 0;
    if (g.work_ptr != nullptr) *g.work_ptr = 0;
    *g.epoch_ptr = epoch;
    __threadfence();
    if (g.comm_progress != nullptr && g.err != nullptr) {
      const uint32_t d = atomicAdd(g.err + 2, 1u) + 1u;
      st_volatile_sys_u32(g.comm_progress + 5, d);
    }
    return true;
  }
  return false;
}

// True when the communicator's abort word is set (polled by every wait on a peer).
__device__ __forceinline__ bool comm_aborted(const GemmArgs& g) { return g.comm_abort != nullptr && *g.comm_abort != 0u; }

struct __align__(8) SharedCtl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  uint32_t epoch;
  volatile uint32_t abort;
};

template <typename Epilogue, int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ GemmArgs g, const __grid_constant__ Epilogue epi) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128B-swizzled tiles.
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  constexpr int NS = Epilogue::kSingleStages;  // ring depth: an epilogue with a large scratch takes a stage
  constexpr int kWarpSmem = Epilogue::kWarpSmemBytes;
  static_assert(NS >= 2 && NS <= kStages, "ring depth");
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + NS * kStageBytes);
  static_assert(sizeof(SharedCtl) <= kCtlBytes, "control block outgrew its slot");
  uint8_t* epi_smem = smem + NS * kStageBytes + kCtlBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int n_gemm = g.n_gemm_ctas > 0 ? g.n_gemm_ctas : static_cast<int>(gridDim.x);
  if (static_cast<int>(blockIdx.x) >= n_gemm) {
    // Communication CTA of a fused kernel: no tensor memory, no tiles.
    __shared__ uint32_t s_epoch;
    __shared__ volatile uint32_t s_abort;
    if (threadIdx.x == 0) {
      s_epoch = g.epoch_ptr ? *g.epoch_ptr + 1u : 1u;
      s_abort = 0;
      fused_kernel_started(g);
    }
    __syncthreads();
    epi.comm_cta(g, s_epoch, static_cast<int>(blockIdx.x) - n_gemm, static_cast<int>(gridDim.x) - n_gemm, &s_abort, smem, base);
    __syncthreads();
    if (threadIdx.x == 0) {
      report_failure(g, s_abort);
      if (finish_epoch(g, s_epoch)) epi.last_cta_out(g, s_epoch);
    }
    return;
  }
  const int tiles_m = (g.M + kBM - 1) / kBM;
  static_assert(BN % 32 == 0 && BN >= 64 && BN <= kBN, "tile width: a multiple of 32 up to 256");
  const int tiles_n = (g.N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (g.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[b]), kEpilogueWarps);
    }
    ctl->abort = 0;
    ctl->epoch = g.epoch_ptr ? *g.epoch_ptr + 1u : 1u;
    fused_kernel_started(g);
    fence_barrier_init();
    fence_proxy_async();
  }
  if (warp == 0 && lane == 0) {
    prefetch_tensormap(&tma_a);
    prefetch_tensormap(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t epoch = ctl->epoch;
  const uint64_t budget = g.wait_budget_ns;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;  // ring position over all k-blocks of all my tiles
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += n_gemm) {
        int tm, tn;
        tile_coords(g, t, tiles_m, tiles_n, &tm, &tn);
        // all-gather -> GEMM: the rows of this tile may still be on their way
        if (g.a_ready != nullptr) {
          const int chunk = (tm * kBM) / g.rows_per_chunk;
          const int last_chunk = (min(tm * kBM + kBM, g.M) - 1) / g.rows_per_chunk;
          const uint32_t target = epoch * g.a_ready_mult;
          bool waited = false;
          for (int c = chunk; c <= last_chunk && ok; ++c) {
            if (c >= g.a_local_first && c < g.a_local_first + g.a_local_count) continue;  // rows that never left this GPU
            waited = true;
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (static_cast<int32_t>(ld_acquire_sys_u32(g.a_ready + c) - target) < 0) {
              if ((++spins & 255u) == 0u) {
                const bool aborted = comm_aborted(g);
                if (aborted || ctl->abort != 0u || globaltimer_ns() - t0 > budget) {
                  if (ctl->abort == 0u) ctl->abort = aborted ? kGemmAborted : kGemmRowsTimeout;
                  ok = false;
                  break;
                }
              }
            }
          }
          if (!ok) break;
          // rows written by a peer's generic stores are about to be read by the async proxy
          if (waited) asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % NS;
          const uint32_t ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1u, &ctl->abort, budget)) { ok = false; break; }
          const uint32_t full = smem_u32(&ctl->full[s]);
          mbar_arrive_expect_tx(full, kTileABytes + BN * kBK * 2);
          const uint32_t sa = base + s * kStageBytes;
          tma_load_2d(sa, &tma_a, full, kb * kBK, tm * kBM);
          tma_load_2d(sa + kTileABytes, &tma_b, full, kb * kBK, tn * BN);
        }
      }
      // Wind-down after a failed wait: let copies that are still in flight land
      // before the CTA (and its shared memory) goes away.
      if (!ok) {
        for (uint32_t back = 0; back < NS && back < it; ++back) {
          const uint32_t j = it - 1 - back;
          mbar_wait(smem_u32(&ctl->full[j % NS]), (j / NS) & 1u, &ctl->abort /*already set*/, 0);
          // (budget 0: one more try each; the data either landed or the MMA side consumed it)
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, BN);
      uint32_t it = 0;
      uint32_t local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += n_gemm, ++local) {
        const uint32_t buf = local & 1u;
        const uint32_t acc_ph = (local >> 1) & 1u;
        if (!mbar_wait(smem_u32(&ctl->tmem_empty[buf]), acc_ph ^ 1u, &ctl->abort, budget)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * kBN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % NS;
          const uint32_t ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&ctl->full[s]), ph, &ctl->abort, budget)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = base + s * kStageBytes;
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + kTileABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            // advance 16 elements = 32 bytes inside the 128-byte swizzle row: +2 in the address field
            umma_bf16(d, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2), idesc,
                      (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(smem_u32(&ctl->empty[s]));  // the stage is free once these MMAs have read it
        }
        if (ok) umma_commit(smem_u32(&ctl->tmem_full[buf]));
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;  // TMEM lane quarter this warp may access
    uint8_t* warp_smem = epi_smem + (warp - 2) * kWarpSmem;
    epi.warp_begin(warp_smem, lane);
    uint32_t local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += n_gemm, ++local) {
      int tm, tn;
      tile_coords(g, t, tiles_m, tiles_n, &tm, &tn);
      const uint32_t buf = local & 1u;
      const uint32_t acc_ph = (local >> 1) & 1u;
      if (!mbar_wait(smem_u32(&ctl->tmem_full[buf]), acc_ph, &ctl->abort, budget)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = tm * kBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kBN;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        epi.store(g, epoch, row, tn * BN + c * 32, r, c, warp_smem, lane);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[buf]));
      epi.tile_done(g, epoch, tm, tn, q, lane, warp_smem);
    }
    epi.after_tiles(g, epoch, static_cast<int>(blockIdx.x), n_gemm, q, lane, &ctl->abort, warp_smem);
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    report_failure(g, ctl->abort);
    if (finish_epoch(g, epoch)) epi.last_cta_out(g, epoch);
  }
}

constexpr int kMaxDevices = 64;
inline int current_device_slot() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) (void)cudaGetLastError();
  return (dev >= 0 && dev < kMaxDevices) ? dev : 0;
}

template <typename Epilogue, int BN>
inline cudaError_t launch_bn(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const Epilogue& epi, int grid,
                             cudaStream_t stream) {
  auto kernel = gemm_bf16_kernel<Epilogue, BN>;
  constexpr int smem_bytes = Epilogue::kSingleStages * kStageBytes + 1024 /*alignment slack*/ + kCtlBytes +
                             kEpilogueWarps * Epilogue::kWarpSmemBytes;
  static_assert(smem_bytes <= 227 * 1024, "shared memory of the single-CTA kernel");
  static bool configured[kMaxDevices] = {};  // the attribute belongs to the function on ONE device
  const int dev = current_device_slot();
  if (!configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  kernel<<<grid, kThreads, smem_bytes, stream>>>(ta, tb, g, epi);
  return cudaGetLastError();
}

// `bn` is the tile width the B tensor map was built for: 256, 224, 192 or 128.
template <typename Epilogue>
inline cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const Epilogue& epi, int grid,
                          cudaStream_t stream, int bn = kBN) {
  switch (bn) {
    case 256: return launch_bn<Epilogue, 256>(ta, tb, g, epi, grid, stream);
    case 224: return launch_bn<Epilogue, 224>(ta, tb, g, epi, grid, stream);
    case 192: return launch_bn<Epilogue, 192>(ta, tb, g, epi, grid, stream);
    case 128: return launch_bn<Epilogue, 128>(ta, tb, g, epi, grid, stream);
  }
  return cudaErrorInvalidValue;
}

}  // namespace gemm
}  // namespace mnccl
