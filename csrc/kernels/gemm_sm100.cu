// bf16 GEMM for sm_100a on the 5th-generation tensor cores, written by hand:
//   C[M,N] = A[M,K] * B[N,K]^T      (A, B row-major / "K-major", fp32 accumulate)
// One persistent CTA per SM, warp-specialised:
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of A (128 x 64) and
//               B (256 x 64) into a 4-stage shared-memory ring (128B swizzle)
//   warp 1      MMA issuer: one thread issues tcgen05.mma 128x256x16 from the
//               shared-memory descriptors into tensor memory; tcgen05.commit
//               releases ring stages and publishes finished accumulators
//   warps 2-5   epilogue: tcgen05.ld the fp32 accumulators (TMEM lanes = rows),
//               convert, store; two 256-column accumulators alternate so the
//               epilogue of one tile overlaps the MMAs of the next
// The same kernel body serves the tensor-parallel fused paths through two
// optional hooks: rows of A that become valid chunk by chunk (all-gather ->
// GEMM) and an epilogue that pushes partial tiles to the rank that owns the
// rows (GEMM -> reduce-scatter); see gemm_fused.cu.
//
// Every wait is bounded: a wait that runs out sets a flag, all roles wind down,
// tensor memory is freed and the kernel reports an error word to the host.
// The reference has no GEMM and no tensor-core code; this exists because the
// tensor-parallel workload fuses it with the collectives of this library.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <mutex>

#include "kernels/gemm_sm100.h"
#include "kernels/sm100_ptx.cuh"
#include "mem/cuda_driver.h"

namespace mnccl {
namespace gemm {

using namespace sm100;

namespace {

// -------------------------------------------------------------------- device

__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct __align__(8) SharedCtl {
  uint64_t full[kStages];
  uint64_t empty[kStages];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint32_t tmem_base;
  volatile uint32_t abort;
};

template <typename Epilogue>
__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ GemmArgs g, const __grid_constant__ Epilogue epi) {
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment for the 128B-swizzled tiles.
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (base - raw);
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(smem + kStages * kStageBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (g.M + kBM - 1) / kBM;
  const int tiles_n = (g.N + kBN - 1) / kBN;
  const int num_tiles = tiles_m * tiles_n;
  const int num_kb = (g.K + kBK - 1) / kBK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&ctl->full[s]), 1);
      mbar_init(smem_u32(&ctl->empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&ctl->tmem_full[b]), 1);
      mbar_init(smem_u32(&ctl->tmem_empty[b]), kEpilogueWarps);
    }
    ctl->abort = 0;
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
  const uint64_t budget = g.wait_budget_ns;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;  // ring position over all k-blocks of all my tiles
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
        int tm, tn;
        tile_coords(g, t, tiles_m, tiles_n, &tm, &tn);
        // all-gather -> GEMM: the rows of this tile may still be on their way
        if (g.a_ready != nullptr) {
          const int chunk = (tm * kBM) / g.rows_per_chunk;
          const int last_chunk = (min(tm * kBM + kBM, g.M) - 1) / g.rows_per_chunk;
          for (int c = chunk; c <= last_chunk && ok; ++c) {
            const uint64_t t0 = globaltimer_ns();
            uint32_t spins = 0;
            while (static_cast<int32_t>(ld_acquire_gpu(g.a_ready + c) - g.a_epoch) < 0) {
              if ((++spins & 255u) == 0u && (ctl->abort != 0u || globaltimer_ns() - t0 > budget)) {
                ctl->abort = 2u;
                ok = false;
                break;
              }
            }
          }
          if (!ok) break;
          // data written by other SMs' generic stores, read by the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
          if (!mbar_wait(smem_u32(&ctl->empty[s]), ph ^ 1u, &ctl->abort, budget)) { ok = false; break; }
          const uint32_t full = smem_u32(&ctl->full[s]);
          mbar_arrive_expect_tx(full, kStageBytes);
          const uint32_t sa = base + s * kStageBytes;
          tma_load_2d(sa, &tma_a, full, kb * kBK, tm * kBM);
          tma_load_2d(sa + kTileABytes, &tma_b, full, kb * kBK, tn * kBN);
        }
      }
      // Wind-down after a failed wait: let copies that are still in flight land
      // before the CTA (and its shared memory) goes away.
      if (!ok) {
        for (uint32_t back = 0; back < kStages && back < it; ++back) {
          const uint32_t j = it - 1 - back;
          mbar_wait(smem_u32(&ctl->full[j % kStages]), (j / kStages) & 1u, &ctl->abort /*already set*/, 0);
          // (budget 0: one more try each; the data either landed or the MMA side consumed it)
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(kBM, kBN);
      uint32_t it = 0;
      uint32_t local = 0;
      bool ok = true;
      for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
        const uint32_t buf = local & 1u;
        const uint32_t acc_ph = (local >> 1) & 1u;
        if (!mbar_wait(smem_u32(&ctl->tmem_empty[buf]), acc_ph ^ 1u, &ctl->abort, budget)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d = tmem_base + buf * kBN;
        for (int kb = 0; kb < num_kb; ++kb, ++it) {
          const uint32_t s = it % kStages;
          const uint32_t ph = (it / kStages) & 1u;
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
    uint32_t local = 0;
    bool ok = true;
    for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++local) {
      int tm, tn;
      tile_coords(g, t, tiles_m, tiles_n, &tm, &tn);
      const uint32_t buf = local & 1u;
      const uint32_t acc_ph = (local >> 1) & 1u;
      if (!mbar_wait(smem_u32(&ctl->tmem_full[buf]), acc_ph, &ctl->abort, budget)) { ok = false; break; }
      tc_fence_after_sync();
      const int row = tm * kBM + q * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + buf * kBN;
#pragma unroll 1
      for (int c = 0; c < kBN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        epi.store(g, row, tn * kBN + c * 32, r, tm, tn);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(smem_u32(&ctl->tmem_empty[buf]));
      epi.tile_done(g, tm, tn, q, lane);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
  if (threadIdx.x == 0 && ctl->abort != 0u && g.err != nullptr) atomicCAS(g.err, 0u, ctl->abort);
}

}  // namespace

// -------------------------------------------------------------------- host

namespace {

std::mutex g_mu;
uint32_t* g_err_dev = nullptr;  // one error word per process and device (device 0..15)
int g_err_device = -1;

}  // namespace

bool make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                          uint32_t box_rows, uint32_t box_cols, std::string* why) {
  const CudaDriver* d = CudaDriver::get();
  if (!d || !d->TensorMapEncodeTiled) {
    if (why) *why = "cuTensorMapEncodeTiled unavailable";
    return false;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_elems * 2) % 16 != 0) {
    if (why) *why = "operand base and row stride must be 16-byte aligned";
    return false;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = d->TensorMapEncodeTiled(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                                       estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    if (why) *why = "cuTensorMapEncodeTiled: " + d->error_string(r);
    return false;
  }
  return true;
}

uint32_t* error_word() {
  std::lock_guard<std::mutex> lk(g_mu);
  int dev = 0;
  cudaGetDevice(&dev);
  if (g_err_dev == nullptr || g_err_device != dev) {
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64);
    g_err_dev = p;  // (a word allocated for another device stays allocated; processes here use one device)
    g_err_device = dev;
  }
  return g_err_dev;
}

int sm_count() {
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  return sms;
}

template <typename Epilogue>
cudaError_t launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, const Epilogue& epi, int grid,
                   cudaStream_t stream) {
  auto kernel = gemm_bf16_kernel<Epilogue>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return e;
    configured = true;
  }
  kernel<<<grid, kThreads, kSmemBytes, stream>>>(ta, tb, g, epi);
  return cudaGetLastError();
}

template cudaError_t launch<StoreEpilogue<false>>(const CUtensorMap&, const CUtensorMap&, const GemmArgs&,
                                                  const StoreEpilogue<false>&, int, cudaStream_t);
template cudaError_t launch<StoreEpilogue<true>>(const CUtensorMap&, const CUtensorMap&, const GemmArgs&,
                                                 const StoreEpilogue<true>&, int, cudaStream_t);

}  // namespace gemm
}  // namespace mnccl

using namespace mnccl;
using namespace mnccl::gemm;

extern "C" {
#define MNCCL_EXPORT __attribute__((visibility("default")))

// C[M,N] = A[M,K] * B[N,K]^T, bf16 operands, fp32 accumulation.
// out_f32 = 0: C is bf16; 1: C is fp32.  lda / ldb / ldc are row strides in
// elements (0 = dense).  Requirements: A, B 16-byte aligned, lda and ldb
// multiples of 8, K >= 8.  Returns 0, or a negative code for bad arguments, or
// a cudaError_t + 1000.
MNCCL_EXPORT int mncclGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                               int out_f32, cudaStream_t stream) {
  if (!A || !B || !C || M <= 0 || N <= 0 || K <= 0) return -1;
  if (lda == 0) lda = K;
  if (ldb == 0) ldb = K;
  if (ldc == 0) ldc = N;
  if (lda < K || ldb < K || ldc < N) return -2;
  CUtensorMap ta, tb;
  std::string why;
  if (!make_tensor_map_bf16(&ta, A, M, K, lda, kBM, kBK, &why) || !make_tensor_map_bf16(&tb, B, N, K, ldb, kBN, kBK, &why)) {
    fprintf(stderr, "[Mini-NCCL] GEMM: %s\n", why.c_str());
    return -3;
  }
  GemmArgs g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.c = C;
  g.ldc = ldc;
  g.err = error_word();
  g.wait_budget_ns = 2000000000ull;
  g.group_m = 8;
  const int tiles = ((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
  const int grid = tiles < sm_count() ? tiles : sm_count();
  cudaError_t e = out_f32 ? launch(ta, tb, g, StoreEpilogue<true>{}, grid, stream)
                          : launch(ta, tb, g, StoreEpilogue<false>{}, grid, stream);
  return e == cudaSuccess ? 0 : static_cast<int>(e) + 1000;
}

// Reads and clears the GEMM error word of the current device (0 = no bounded
// wait ever ran out).  Synchronises the device.
MNCCL_EXPORT int mncclGemmStatus(uint32_t* status) {
  uint32_t* w = error_word();
  if (!w || !status) return -1;
  if (cudaDeviceSynchronize() != cudaSuccess) return -2;
  if (cudaMemcpy(status, w, 4, cudaMemcpyDeviceToHost) != cudaSuccess) return -2;
  cudaMemset(w, 0, 4);
  return 0;
}

}  // extern "C"
