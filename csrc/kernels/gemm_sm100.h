// Shared definitions of the sm_100a bf16 GEMM (tile shape, arguments, the
// epilogue interface) used by gemm_sm100.cu and the fused kernels.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

namespace mnccl {
namespace gemm {

constexpr int kBM = 128;          // tile rows  (UMMA M; TMEM lanes)
constexpr int kBN = 256;          // widest tile (UMMA N; TMEM columns per accumulator); 224 and 192 are used
                                 // when they cut the number of waves (shared memory is laid out for 256)
constexpr int kBK = 64;           // k-block: 64 bf16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;        // K of one tcgen05.mma for 16-bit types
constexpr int kStages = 4;
constexpr int kTileABytes = kBM * kBK * 2;           // 16 KB
constexpr int kTileBBytes = kBN * kBK * 2;           // 32 KB
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kTmemCols = 512;    // two fp32 accumulators of 256 columns
constexpr int kEpilogueWarps = 4;
constexpr int kThreads = 32 * (2 + kEpilogueWarps);
constexpr int kCtlBytes = 256;            // barriers and control words
constexpr int kEpiRowBytes = 128 + 16;    // 64 bf16 of one row + padding against bank conflicts
constexpr int kEpiWarpBytes = 32 * kEpiRowBytes;  // per epilogue warp: 32 rows x 64 columns, for transposed stores

struct GemmArgs {
  int M, N, K;
  void* c;                 // output (StoreEpilogue)
  int ldc;
  int group_m;             // tile rasterisation: group of m-tiles that share B tiles in L2
  uint32_t* err;           // device error word (first failed wait)
  uint64_t wait_budget_ns;
  // all-gather -> GEMM: chunk c of A's rows is valid once a_ready[c] >= epoch * a_ready_mult;
  // chunks [a_local_first, a_local_first + a_local_count) are local and need no wait.
  const uint32_t* a_ready;
  uint32_t a_ready_mult;
  int rows_per_chunk;
  int a_local_first, a_local_count;
  int m_tile_rotate;       // first m-tile to compute (so that local rows go first)
  // fused kernels: CTAs [0, n_gemm_ctas) compute tiles, the rest run the epilogue's
  // comm_cta(); 0 means every CTA computes.
  int n_gemm_ctas;
  // Device-resident call counter of the fused op: the kernel works with epoch = *epoch_ptr + 1
  // and its last CTA (ticket) stores it back, so a captured launch replays correctly.
  uint32_t* epoch_ptr;
  uint32_t* ticket_ptr;
  uint32_t* work_ptr;    // optional work counter of an epilogue, cleared by the last CTA out
  // The communicator's failure model (null for the plain GEMM): its host-mapped abort word, which
  // every wait on a peer polls, and its host-mapped progress words {.., status, detail, started, done}
  // at indices 2..5, through which a failed wait and the kernel's start / end reach the watchdog.
  const volatile uint32_t* comm_abort;
  volatile uint32_t* comm_progress;
  // Split-K of the last, partial wave of the CTA-pair kernel (plain store epilogue only; 0 = off).
  // Work items [0, split_first) are whole 256 x 256 tiles; each of the remaining tiles is cut along K
  // into split_s slices of split_kb k-blocks, one work item each, so that the pairs a partial wave would
  // leave idle share its tiles.  A slice's fp32 accumulators go to split_ws; the last epilogue warp to
  // arrive for its 32 rows (split_cnt) adds the slices IN SLICE ORDER and stores the result.
  int split_first, split_s, split_kb;
  float* split_ws;
  uint32_t* split_cnt;
};

// One unit of work of the pair kernel: a whole tile, or one K-slice of a tile of the last wave.
struct PairWork {
  int tile, kb0, kb1, slice;
  bool split;
};
__host__ __device__ __forceinline__ int pair_work_items(const GemmArgs& g, int num_tiles) {
  return g.split_s > 1 ? g.split_first + (num_tiles - g.split_first) * g.split_s : num_tiles;
}
__host__ __device__ __forceinline__ PairWork pair_work(const GemmArgs& g, int t, int num_kb) {
  PairWork w;
  if (g.split_s <= 1 || t < g.split_first) {
    w.tile = t; w.kb0 = 0; w.kb1 = num_kb; w.slice = 0; w.split = false;
  } else {
    const int u = t - g.split_first;
    w.tile = g.split_first + u / g.split_s;
    w.slice = u % g.split_s;
    w.kb0 = w.slice * g.split_kb;
    w.kb1 = w.kb0 + g.split_kb < num_kb ? w.kb0 + g.split_kb : num_kb;
    w.split = true;
  }
  return w;
}

// Codes a CTA leaves in its shared abort flag (and the device error word).
enum GemmAbort : uint32_t { kGemmOk = 0, kGemmMbarTimeout = 1, kGemmRowsTimeout = 2, kGemmFlagTimeout = 3, kGemmAborted = 4 };

// Tile index -> (tm, tn).  m-tiles are visited in groups of `group_m` so that a
// wave of CTAs reuses the same B tiles from L2; `m_tile_rotate` rotates the
// m order (fused all-gather: rows that are already local first).
__host__ __device__ __forceinline__ void tile_coords(const GemmArgs& g, int t, int tiles_m, int tiles_n, int* tm, int* tn) {
  const int gm = g.group_m > 0 ? g.group_m : 1;
  const int per_group = gm * tiles_n;
  const int group = t / per_group;
  const int first_m = group * gm;
  const int rows_in_group = (tiles_m - first_m) < gm ? (tiles_m - first_m) : gm;
  const int in_group = t % per_group;
  int m = first_m + in_group % rows_in_group;
  *tn = in_group / rows_in_group;
  m += g.m_tile_rotate;
  if (m >= tiles_m) m -= tiles_m;
  *tm = m;
}

// Plain epilogue: convert and store the accumulator tile to C.
template <bool OUT_F32>
struct StoreEpilogue {
  // what the kernels size their shared memory by: scratch per epilogue warp, TMA ring depth of the
  // single-CTA and of the CTA-pair kernel
  static constexpr int kWarpSmemBytes = kEpiWarpBytes;
  static constexpr int kSingleStages = kStages;
  static constexpr int kPairStages = 6;
  // Thread holds row `row`, columns [col, col+32) as fp32 bit patterns.
  // `chunk` counts the 32-column pieces of the tile; `warp_smem` is kEpiWarpBytes of scratch.
  // A lane's own 32 columns are 64 (bf16) or 128 (fp32) bytes of ONE row, so storing straight from
  // registers makes every instruction touch 32 different lines with 16 bytes each.  Where alignment
  // allows (decided for the whole warp), the piece goes through shared memory instead and leaves as
  // whole rows: 4 (bf16) or 8 (fp32) lanes per row, 16 bytes each.
  __device__ __forceinline__ void store(const GemmArgs& g, uint32_t /*epoch*/, int row, int col, const uint32_t (&r)[32],
                                        int /*chunk*/, uint8_t* warp_smem, int lane) const {
    if (col >= g.N) return;  // the same for the whole warp
    constexpr int kElem = OUT_F32 ? 4 : 2;
    const bool whole_rows = col + 32 <= g.N && ((static_cast<size_t>(g.ldc) * kElem) & 15u) == 0 &&
                            (reinterpret_cast<uintptr_t>(g.c) & 15u) == 0;
    if (whole_rows) {
      const int row_base = row - lane;
      if constexpr (OUT_F32) {
        // 128 bytes per row; two passes of 16 rows through the 32 x 144-byte scratch
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          if ((lane >> 4) == half) {
            uint8_t* mine = warp_smem + (lane & 15) * kEpiRowBytes;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              *reinterpret_cast<uint4*>(mine + j * 16) = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 4; ++it) {
            const int rr = it * 4 + (lane >> 3), seg = lane & 7;
            const int grow = row_base + half * 16 + rr;
            if (grow < g.M) {
              const uint4 v = *reinterpret_cast<const uint4*>(warp_smem + rr * kEpiRowBytes + seg * 16);
              *reinterpret_cast<uint4*>(static_cast<float*>(g.c) + static_cast<size_t>(grow) * g.ldc + col + seg * 4) = v;
            }
          }
          __syncwarp();
        }
      } else {
        uint8_t* mine = warp_smem + lane * kEpiRowBytes;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint4 v;
          uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(r[8 * j + 2 * k]), __uint_as_float(r[8 * j + 2 * k + 1]));
            w[k] = *reinterpret_cast<uint32_t*>(&p);
          }
          *reinterpret_cast<uint4*>(mine + j * 16) = v;
        }
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int rr = it * 8 + (lane >> 2), seg = lane & 3;
          const int grow = row_base + rr;
          if (grow < g.M) {
            const uint4 v = *reinterpret_cast<const uint4*>(warp_smem + rr * kEpiRowBytes + seg * 16);
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(g.c) + static_cast<size_t>(grow) * g.ldc + col + seg * 8) = v;
          }
        }
        __syncwarp();
      }
      return;
    }
    if (row >= g.M) return;
    if constexpr (OUT_F32) {
      float* dst = static_cast<float*>(g.c) + static_cast<size_t>(row) * g.ldc + col;
      for (int j = 0; j < 32 && col + j < g.N; ++j) dst[j] = __uint_as_float(r[j]);
    } else {
      __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(g.c) + static_cast<size_t>(row) * g.ldc + col;
      for (int j = 0; j < 32 && col + j < g.N; ++j) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
    }
  }
  __device__ __forceinline__ void warp_begin(uint8_t*, int) const {}
  __device__ __forceinline__ void tile_done(const GemmArgs&, uint32_t, int, int, int, int, uint8_t*) const {}
  __device__ __forceinline__ void after_tiles(const GemmArgs&, uint32_t, int, int, int, int, volatile uint32_t*, uint8_t*) const {}
  __device__ __forceinline__ void comm_cta(const GemmArgs&, uint32_t, int, int, volatile uint32_t*, uint8_t*, uint32_t) const {}
  __device__ __forceinline__ void last_cta_out(const GemmArgs&, uint32_t) const {}
};

bool make_tensor_map_bf16(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems,
                          uint32_t box_rows, uint32_t box_cols, std::string* why);
uint32_t* error_word();
int sm_count();
int pair_mode();
void set_pair_mode(int mode);

// Tile width (256, 224 or 192; `allow_224` false for epilogues that work on pairs of 32-column
// pieces) that minimises waves x per-tile cost for an M x N problem on `ctas` CTAs.
int pick_tile_n(int M, int N, int ctas, bool allow_224);
// Whether the CTA-pair kernel (256 x 256 tiles on two SMs) should compute an M x N product on
// `ctas` CTAs: never when switched off or when the shape does not divide into pair tiles; in
// automatic mode when the pair tiles fill the SM pairs about as well as single tiles fill the SMs.
bool want_pair(int M, int N, int ctas);

}  // namespace gemm
}  // namespace mnccl
