// The CTA-pair variant of the sm_100a bf16 GEMM: two CTAs on neighbouring SMs (a cluster of 2)
// compute one 256 x 256 output tile with tcgen05.mma.cta_group::2.  Each CTA stages only ITS
// 128 rows of A and ITS 128 rows (half of N) of B per k-block -- 32 KB instead of the 48 KB the
// single-CTA kernel needs for half the output -- so a third less operand traffic per FLOP and
// room for a 6-stage ring.  Nothing is multicast: each CTA issues its own plain TMA loads; the
// loads of the second CTA count their bytes on the leader's barrier (.cta_group::2 form).
//
//   both CTAs   warp 0   TMA producer: own A rows, own half of B -> own shared memory;
//                        completion on the LEADER's full barrier
//   leader      warp 1   one thread issues the MMAs for the pair and commits: ring stages are
//                        released in both CTAs, finished accumulators published to both
//   both CTAs   warps 2-5  epilogue of the CTA's own 128 rows (own tensor memory), through the
//                        same Epilogue objects as the single-CTA kernel
//
// Every wait is bounded as in the single-CTA kernel.  The reference has no GEMM.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kernels/gemm_kernel.cuh"

namespace mnccl {
namespace gemm {

constexpr int k2Stages = 6;  // deepest ring; an epilogue may ask for fewer (Epilogue::kPairStages)
constexpr int k2StageBytes = kTileABytes + kBM * kBK * 2;  // A 128 x 64 + this CTA's half of B 128 x 64: 32 KB
template <typename Epilogue>
constexpr int pair_smem_bytes() {
  return Epilogue::kPairStages * k2StageBytes + 1024 + kCtlBytes + kEpilogueWarps * Epilogue::kWarpSmemBytes;
}

struct __align__(8) SharedCtl2 {
  uint64_t full[k2Stages];    // used in the leader: 2 arrivals (one per producer) + 64 KB of bytes
  uint64_t empty[k2Stages];   // one per CTA: released by the leader's commit (multicast to both)
  uint64_t tmem_full[2];      // one per CTA: accumulator ready (commit, multicast to both)
  uint64_t tmem_empty[2];     // used in the leader: 8 arrivals (4 epilogue warps of each CTA)
  uint32_t tmem_base;
  uint32_t epoch;
  volatile uint32_t abort;
};

template <typename Epilogue>
__global__ void __launch_bounds__(kThreads, 1)
gemm2_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                  const __grid_constant__ GemmArgs g, const __grid_constant__ Epilogue epi) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  constexpr int NS = Epilogue::kPairStages;
  constexpr int kWarpSmem = Epilogue::kWarpSmemBytes;
  static_assert(NS >= 2 && NS <= k2Stages, "ring depth");
  SharedCtl2* ctl = reinterpret_cast<SharedCtl2*>(smem + NS * k2StageBytes);
  static_assert(sizeof(SharedCtl2) <= kCtlBytes, "control block outgrew its slot");
  uint8_t* epi_smem = smem + NS * k2StageBytes + kCtlBytes;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0: leader
  const int n_gemm = g.n_gemm_ctas > 0 ? g.n_gemm_ctas : static_cast<int>(gridDim.x);
  if (static_cast<int>(blockIdx.x) >= n_gemm) {
    // communication CTAs of a fused kernel (both CTAs of their cluster take this branch)
    __shared__ uint32_t s_epoch;
    __shared__ volatile uint32_t s_abort;
    if (threadIdx.x == 0) {
      s_epoch = g.epoch_ptr ? *g.epoch_ptr + 1u : 1u;
      s_abort = 0;
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
  const int pair = static_cast<int>(blockIdx.x) >> 1;
  const int n_pairs = n_gemm >> 1;
  const int tiles_m2 = (g.M + 2 * kBM - 1) / (2 * kBM);  // 256-row tiles
  const int tiles_n = (g.N + kBN - 1) / kBN;
  const int num_tiles = tiles_m2 * tiles_n;
  const int num_kb = (g.K + kBK - 1) / kBK;
  const int num_items = pair_work_items(g, num_tiles);  // tiles, the last wave's cut into K-slices

  if (threadIdx.x == 0) {
    for (int s = 0; s < NS; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 2);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[b]), 2 * kEpilogueWarps);
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
    tmem_alloc_pair(smem_u32(&ctl->tmem_base), kTmemCols);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // the partner's barriers exist before anything arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  const uint32_t epoch = ctl->epoch;
  const uint64_t budget = g.wait_budget_ns;

  // 256-row tile index -> (tm2, tn); this CTA's 128 rows are tile 2 * tm2 + cta of the
  // 128-row numbering the epilogues use.
  GemmArgs g2 = g;
  g2.group_m = g.group_m > 1 ? g.group_m / 2 : 1;
  g2.m_tile_rotate = g.m_tile_rotate / 2;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int t = pair; t < num_items && ok; t += n_pairs) {
        const PairWork w = pair_work(g, t, num_kb);
        int tm2, tn;
        tile_coords(g2, w.tile, tiles_m2, tiles_n, &tm2, &tn);
        const int tm = tm2 * 2 + static_cast<int>(cta);
        if (g.a_ready != nullptr) {
          const int chunk = (tm * kBM) / g.rows_per_chunk;
          const int last_chunk = (min(tm * kBM + kBM, g.M) - 1) / g.rows_per_chunk;
          const uint32_t target = epoch * g.a_ready_mult;
          bool waited = false;
          for (int c = chunk; c <= last_chunk && ok; ++c) {
            if (c >= g.a_local_first && c < g.a_local_first + g.a_local_count) continue;
            waited = true;
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (static_cast<int32_t>(ld_acquire_sys_u32(g.a_ready + c) - target) < 0) {
              if ((++spins & 255u) == 0u && (comm_aborted(g) || ctl->abort != 0u || globaltimer_ns() - t0 > budget)) {
                if (ctl->abort == 0u) ctl->abort = comm_aborted(g) ? kGemmAborted : kGemmRowsTimeout;
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          if (waited) asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const uint32_t s = it % NS;
          const uint32_t ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1u, &ctl->abort, budget)) { ok = false; break; }
          const uint32_t leader_full = map_to_cta(smem_u32(&ctl->full[s]), 0);
          mbar_arrive_expect_tx_cluster(leader_full, k2StageBytes);
          const uint32_t sa = base + s * k2StageBytes;
          tma_load_2d_pair(sa, &tma_a, leader_full, kb * kBK, tm * kBM);
          tma_load_2d_pair(sa + kTileABytes, &tma_b, leader_full, kb * kBK, tn * kBN + static_cast<int>(cta) * (kBN / 2));
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && cta == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(2 * kBM, kBN);
      uint32_t it = 0, local = 0;
      bool ok = true;
      for (int t = pair; t < num_items && ok; t += n_pairs, ++local) {
        const PairWork w = pair_work(g, t, num_kb);
        const uint32_t buf = local & 1u;
        const uint32_t acc_ph = (local >> 1) & 1u;
        if (!mbar_wait(smem_u32(&ctl->tmem_empty[buf]), acc_ph ^ 1u, &ctl->abort, budget)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * kBN;
        for (int kb = w.kb0; kb < w.kb1; ++kb, ++it) {
          const uint32_t s = it % NS;
          const uint32_t ph = (it / NS) & 1u;
          if (!mbar_wait(smem_u32(&ctl->full[s]), ph, &ctl->abort, budget)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t sa = base + s * k2StageBytes;
          const uint64_t da = make_smem_desc_sw128(sa);
          const uint64_t db = make_smem_desc_sw128(sa + kTileABytes);
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k)
            umma_bf16_pair(d, da + static_cast<uint64_t>(k * 2), db + static_cast<uint64_t>(k * 2), idesc,
                           ((kb - w.kb0) | k) != 0 ? 1u : 0u);
          umma_commit_pair(smem_u32(&ctl->empty[s]), 3);  // the stage is free in both CTAs
        }
        if (ok) umma_commit_pair(smem_u32(&ctl->tmem_full[buf]), 3);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own rows)
    const int q = warp & 3;
    uint8_t* warp_smem = epi_smem + (warp - 2) * kWarpSmem;
    epi.warp_begin(warp_smem, lane);
    uint32_t local = 0;
    bool ok = true;
    for (int t = pair; t < num_items && ok; t += n_pairs, ++local) {
      const PairWork w = pair_work(g, t, num_kb);
      int tm2, tn;
      tile_coords(g2, w.tile, tiles_m2, tiles_n, &tm2, &tn);
      const int tm = tm2 * 2 + static_cast<int>(cta);
      const uint32_t buf = local & 1u;
      const uint32_t acc_ph = (local >> 1) & 1u;
      if (!mbar_wait(smem_u32(&ctl->tmem_full[buf]), acc_ph, &ctl->abort, budget)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = tm * kBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kBN;
      if (!w.split) {
#pragma unroll 1
        for (int c = 0; c < kBN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          epi.store(g, epoch, row, tn * kBN + c * 32, r, c, warp_smem, lane);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->tmem_empty[buf]), 0));
        if (tm * kBM < g.M) epi.tile_done(g, epoch, tm, tn, q, lane, warp_smem);
        continue;
      }
      // ---- one K-slice of a tile of the last wave: accumulators -> workspace, laid out so that a store
      // instruction of the warp writes 512 contiguous bytes: float4 index ((c * 8 + j) * 32 + lane)
      constexpr int kQuarterF4 = (kBN / 32) * 8 * 32;               // float4 per (slice, 32-row quarter): 32 KB
      const int tile_r = w.tile - g.split_first;
      const int quarter = (tile_r * 2 + static_cast<int>(cta)) * 4 + q;  // this warp's 32 rows of this tile
      float4* mine = reinterpret_cast<float4*>(g.split_ws) + (static_cast<size_t>(quarter) * g.split_s + w.slice) * kQuarterF4;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          mine[(c * 8 + j) * 32 + lane] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                      __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&ctl->tmem_empty[buf]), 0));
      // All slices of a tile are in flight at once (they form one wave by construction), so the warps that
      // hold the same 32 rows may wait for one another: when every slice has been delivered, slice s adds
      // up, IN SLICE ORDER, the 32-column pieces c = s, s + slices, ... and stores them.  (Leaving the sum
      // to the last warp to arrive made one warp read all slices: 16 x 32 KB at one warp's L2 rate cost
      // more than the wave the split saves.)
      const int slices = (num_kb + g.split_kb - 1) / g.split_kb;
      uint32_t* cnt = g.split_cnt + quarter;
      bool all_in = true;
      if (lane == 0) {
        __threadfence();
        atomicAdd(cnt, 1u);
        const uint64_t t0 = globaltimer_ns();
        uint32_t spins = 0;
        while (ld_acquire_sys_u32(cnt) < static_cast<uint32_t>(slices)) {
          if ((++spins & 255u) == 0u && (ctl->abort != 0u || globaltimer_ns() - t0 > budget)) {
            if (ctl->abort == 0u) ctl->abort = kGemmFlagTimeout;
            all_in = false;
            break;
          }
        }
      }
      all_in = __shfl_sync(0xffffffffu, all_in ? 1 : 0, 0) != 0;
      if (!all_in) { ok = false; break; }
      const float4* all = reinterpret_cast<const float4*>(g.split_ws) + static_cast<size_t>(quarter) * g.split_s * kQuarterF4;
#pragma unroll 1
      for (int c = w.slice; c < kBN / 32; c += slices) {
        float acc[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
#pragma unroll 2
        for (int sl = 0; sl < slices; ++sl) {
          float4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = __ldcg(all + static_cast<size_t>(sl) * kQuarterF4 + (c * 8 + j) * 32 + lane);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc[4 * j] += v[j].x; acc[4 * j + 1] += v[j].y; acc[4 * j + 2] += v[j].z; acc[4 * j + 3] += v[j].w;
          }
        }
        uint32_t r[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(acc[i]);
        epi.store(g, epoch, row, tn * kBN + c * 32, r, c, warp_smem, lane);
      }
      // the last reader leaves the counter clean for the next launch
      __syncwarp();
      if (lane == 0 && atomicAdd(cnt, 1u) == static_cast<uint32_t>(2 * slices - 1)) *cnt = 0;
      if (w.slice == 0 && tm * kBM < g.M) epi.tile_done(g, epoch, tm, tn, q, lane, warp_smem);
    }
    // the single-CTA numbering of CTAs for the epilogues' follow-up pass
    epi.after_tiles(g, epoch, static_cast<int>(blockIdx.x), n_gemm, q, lane, &ctl->abort, warp_smem);
  }

  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves (or frees tensor memory) while its partner may still signal it
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0) {
    report_failure(g, ctl->abort);
    if (finish_epoch(g, epoch)) epi.last_cta_out(g, epoch);
  }
}

// Launch with clusters of two CTAs.  `grid` must be even; it is cut down to the number of CTA pairs
// the device can hold at once (a GPC with an odd number of free SMs leaves one unpaired), because a
// persistent kernel must never need a second round of CTAs.
template <typename Epilogue>
inline cudaError_t launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const Epilogue& epi,
                               int grid, cudaStream_t stream, int* grid_used = nullptr) {
  auto kernel = gemm2_bf16_kernel<Epilogue>;
  static bool configured_dev[kMaxDevices] = {};
  static int max_clusters_dev[kMaxDevices] = {};
  const int dev = current_device_slot();
  bool& configured = configured_dev[dev];
  int& max_clusters = max_clusters_dev[dev];
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pair_smem_bytes<Epilogue>();
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_bytes<Epilogue>());
    if (e != cudaSuccess) return e;
    cfg.gridDim = dim3(2 * 74);
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kernel, &cfg);
    if (e != cudaSuccess || max_clusters <= 0) {
      (void)cudaGetLastError();
      max_clusters = 64;  // conservative
    }
    configured = true;
  }
  if (grid > 2 * max_clusters) grid = 2 * max_clusters;
  cfg.gridDim = dim3(grid);
  if (grid_used) *grid_used = grid;
  return cudaLaunchKernelEx(&cfg, kernel, ta, tb, g, epi);
}

// Number of CTA pairs of this kernel the device can hold at once (asked once per kernel).
template <typename Epilogue>
inline int max_pairs() {
  static int cached_dev[kMaxDevices] = {};
  int& cached = cached_dev[current_device_slot()];
  if (cached > 0) return cached;
  auto kernel = gemm2_bf16_kernel<Epilogue>;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * 74);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = pair_smem_bytes<Epilogue>();
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem_bytes<Epilogue>()) != cudaSuccess ||
      cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) {
    (void)cudaGetLastError();
    n = 64;
  }
  cached = n;
  return n;
}

}  // namespace gemm
}  // namespace mnccl
