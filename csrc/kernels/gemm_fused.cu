// Tensor-parallel fusions of the sm_100a GEMM with its collective, each ONE kernel:
//
//   GEMM -> reduce-scatter.  Every rank multiplies its K-slice: P_r = A_r * B_r^T, [M, N];
//   the result row block i belongs to rank i.  The epilogue converts each 128 x 256
//   accumulator tile to bf16 and stores it straight into the OWNER's staging slot for
//   this source rank over NVLink (plain peer stores), then raises a per-tile flag
//   there (st.release.sys).  Tiles are visited owner by owner starting with the next
//   rank, the local rows last, so the transfers overlap the remaining math.  When a
//   CTA has no tiles left, its epilogue warps turn to the rows this rank owns: they
//   wait (bounded) for the flags of all ranks, add the partial tiles in rank order in
//   fp32 and write the bf16 result.  Deterministic; nothing is reduced in the switch.
//   Second form, where the staging has an NVSwitch multicast mapping (RsEpilogue::mc_stage):
//   the bf16 tiles stay in the rank's OWN staging, every rank walks the tiles in the same
//   order, the flag still goes to the owner, and a few CTAs of the owner (joined by the
//   others as they run out of tiles) read the sum of all ranks' copies with
//   multimem.ld_reduce while the remaining tiles are computed: the owner receives M / R
//   reduced rows instead of R - 1 partial copies; the switch orders the sum.
//
//   all-gather -> GEMM.  X is sharded by rows; every rank needs all of X times its own
//   weight slice.  The local shard already sits at its place inside the gather buffer.
//   A few CTAs of the grid do no math: once every peer has left its previous call they push the local
//   shard into every peer's gather buffer (peer stores), chunk of 128 rows by chunk,
//   and count each finished chunk into the peer's ready counters (red.release.sys).
//   The GEMM CTAs start on the local rows at once; their TMA producer waits (bounded)
//   for a chunk's counter before loading tiles of those rows -- always from local
//   memory, never from a peer.
//
// Call counters (epochs) are device-resident, flags and counters only grow, staging
// alternates between two halves: no clearing between calls and a captured launch can
// be replayed.  The reference has neither tensor parallelism nor a GEMM; these kernels
// are what "AllReduce fused with the adjacent compute" means for this library.
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "kernels/comm_dev.h"
#include "kernels/gemm2_kernel.cuh"
#include "kernels/gemm_kernel.cuh"

namespace mnccl {
namespace gemm {

constexpr int kMaxTpRanks = 8;
constexpr int kAgSlots = 16;          // rows in flight per communication CTA (ring in shared memory)
constexpr int kAgPartsPerChunk = 4;   // a 128-row chunk is pushed as four independent quarters

__device__ __forceinline__ void st_release_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void epilogue_warps_sync() {
  // the four epilogue warps (128 threads) on named barrier 1
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// Bounded wait for *p >= target (wrap-safe) with system-scope acquire.  Gives up when the budget runs
// out, when another role of the CTA has given up (*abort_flag) or when the communicator's abort word
// is set (the watchdog of this or of another local rank tripped): the kernel then winds down and the
// failure reaches the communicator through report_failure().
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* p, uint32_t target, volatile uint32_t* abort_flag,
                                              const GemmArgs& g) {
  if (static_cast<int32_t>(ld_acquire_sys_u32(p) - target) >= 0) return true;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(p) - target) >= 0) return true;
    if ((it & 255u) == 0u) {
      if (*abort_flag != 0u) return false;
      if (comm_aborted(g)) {
        *abort_flag = kGemmAborted;
        return false;
      }
      if (globaltimer_ns() - t0 > g.wait_budget_ns) {
        *abort_flag = kGemmFlagTimeout;
        return false;
      }
    }
  }
}

// ------------------------------------------------------------------ GEMM -> reduce-scatter

struct RsEpilogue {
  static constexpr int kWarpSmemBytes = kEpiWarpBytes;
  static constexpr int kSingleStages = kStages;
  static constexpr int kPairStages = 6;
  int rank, nranks;
  int rows_per_rank;                 // M / nranks, a multiple of 128
  char* stage[kMaxTpRanks];          // every rank's staging: [2][nranks sources][local tiles][128 rows][bn] bf16
  uint32_t* flags[kMaxTpRanks];      // every rank's flags:   [nranks][tiles_m_local * tiles_n]
  __nv_bfloat16* out;                // [rows_per_rank, N] on this rank
  int ldo;
  int bn;                            // tile width of this launch (256 or 192)
  int tiled;                         // staging layout: 0 row-major [rows_per_rank][N] (default), 1 tile by tile (MINI_NCCL_RS_TILED=1)
  // Switch mode (mc_stage != null): the partial tiles stay in THIS rank's staging, laid out [2][M][N], and
  // the owner of a row block sums all ranks' copies with one multimem.ld_reduce through the NVSwitch
  // multicast mapping of the staging: a GPU receives M / nranks reduced rows instead of nranks - 1 partial
  // copies, and the sum is taken while the other tiles are still being computed.
  const char* mc_stage;              // multicast address of the staging (same offset on every rank), or null
  uint32_t* work;                    // ticket counter of the reduction items (reset by the last CTA out)

  // One source rank's partial sums of the rows one rank owns.  Row-major by default.  The tiled
  // layout (a 128 x bn tile is one contiguous block) looked better in a two-GPU store test (compact
  // destinations 665 GB/s, 512-byte runs 8 KB apart 340 GB/s) but measured WORSE on 8 GPUs
  // (107 against 89 us on 4096 x 4096 x 1792), so it stays an option.
  __device__ __forceinline__ size_t tile_elems() const { return static_cast<size_t>(kBM) * bn; }
  __device__ __forceinline__ size_t slot_elems(const GemmArgs& g) const {
    return tiled ? static_cast<size_t>(rows_per_rank / kBM) * ((g.N + bn - 1) / bn) * tile_elems()
                 : static_cast<size_t>(rows_per_rank) * g.N;
  }
  // element (row r of the owner's rows, column c) of one source's slot
  __device__ __forceinline__ size_t elem_offset(const GemmArgs& g, int r, int c) const {
    if (!tiled) return static_cast<size_t>(r) * g.N + c;
    const int tiles_n = (g.N + bn - 1) / bn;
    const int ltm = r / kBM, tn = c / bn;
    return (static_cast<size_t>(ltm) * tiles_n + tn) * tile_elems() + static_cast<size_t>(r - ltm * kBM) * bn + (c - tn * bn);
  }

  // Peer stores want long contiguous runs: a warp's 32 rows x 32 columns piece would be 32
  // separate 16-byte writes per instruction.  So two pieces (64 columns = 128 bytes per row) are
  // first laid out row-major in shared memory, then written with 8 lanes per row: every store
  // instruction of the warp covers four full 128-byte lines of the owner's memory.
  __device__ __forceinline__ void store(const GemmArgs& g, uint32_t epoch, int row, int col, const uint32_t (&r)[32],
                                        int chunk, uint8_t* warp_smem, int lane) const {
    uint8_t* mine = warp_smem + lane * kEpiRowBytes + (chunk & 1) * 64;
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
    if ((chunk & 1) == 0) return;
    __syncwarp();
    const int row_base = row - lane;        // first row of this warp's 32
    const int col_base = col - 32;          // first of the 64 columns
    const int owner = row_base / rows_per_rank;   // a 128-row tile never straddles owners
    const bool sw = mc_stage != nullptr;
    __nv_bfloat16* slot = sw ? reinterpret_cast<__nv_bfloat16*>(stage[rank]) + static_cast<size_t>(epoch & 1u) * g.M * g.N
                             : reinterpret_cast<__nv_bfloat16*>(stage[owner]) +
                                   (static_cast<size_t>(epoch & 1u) * nranks + rank) * slot_elems(g);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int rr = it * 4 + (lane >> 3);  // 4 rows per instruction
      const int seg = lane & 7;             // 8 x 16 bytes per row
      const int grow = row_base + rr;
      const int gcol = col_base + seg * 8;
      if (grow < g.M && gcol < g.N) {
        const uint4 v = *reinterpret_cast<const uint4*>(warp_smem + rr * kEpiRowBytes + seg * 16);
        const size_t off = sw ? static_cast<size_t>(grow) * g.N + gcol : elem_offset(g, grow - owner * rows_per_rank, gcol);
        *reinterpret_cast<uint4*>(slot + off) = v;
      }
    }
    __syncwarp();  // the scratch is reused by the next pair of pieces
  }

  // All four epilogue warps call this after the last store of a tile.
  __device__ __forceinline__ void warp_begin(uint8_t*, int) const {}

  __device__ __forceinline__ void tile_done(const GemmArgs& g, uint32_t epoch, int tm, int tn, int q, int lane,
                                            uint8_t* /*warp_smem*/) const {
    epilogue_warps_sync();  // every store of the tile precedes the flag
    if (q == 0 && lane == 0) {
      const int tiles_n = (g.N + bn - 1) / bn;
      const int tiles_m_local = rows_per_rank / kBM;
      const int owner = (tm * kBM) / rows_per_rank;
      const int ltm = tm - owner * tiles_m_local;
      st_release_sys_u32(flags[owner] + (static_cast<size_t>(rank) * tiles_m_local + ltm) * tiles_n + tn, epoch);
    }
  }

  // Reduction of the rows this rank owns, by the epilogue warps of every CTA.  The pass is bound by
  // load latency, so every thread keeps 32 independent 16-byte loads in flight whatever the number
  // of ranks: NR sources x U vectors.
  __device__ __forceinline__ void after_tiles(const GemmArgs& g, uint32_t epoch, int cta, int n_cta, int q, int lane,
                                              volatile uint32_t* abort_flag, uint8_t* /*warp_smem*/) const {
    if (mc_stage != nullptr) {
      reduce_switch<128, false>(g, epoch, ((q + 2) & 3) * 32 + lane, abort_flag);
      return;
    }
    if (nranks <= 1) reduce_owned<1, 16>(g, epoch, cta, n_cta, q, lane, abort_flag);
    else if (nranks <= 2) reduce_owned<2, 16>(g, epoch, cta, n_cta, q, lane, abort_flag);
    else if (nranks <= 4) reduce_owned<4, 8>(g, epoch, cta, n_cta, q, lane, abort_flag);
    else reduce_owned<kMaxTpRanks, 4>(g, epoch, cta, n_cta, q, lane, abort_flag);
  }

  template <int NR, int U>
  __device__ __forceinline__ void reduce_owned(const GemmArgs& g, uint32_t epoch, int cta, int n_cta, int q, int lane,
                                               volatile uint32_t* abort_flag) const {
    const int tiles_n = (g.N + bn - 1) / bn;
    const int tiles_m_local = rows_per_rank / kBM;
    constexpr int kParts = 32 / U, kRows = kBM / kParts;   // an item: 4 * U rows x 256 columns of one tile: one pass of the 128 threads
    const int items = tiles_m_local * tiles_n * kParts;
    const int tid = ((q + 2) & 3) * 32 + lane;        // 0..127 over warps 2,3,4,5 in launch order
    const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(stage[rank]) +
                                static_cast<size_t>(epoch & 1u) * nranks * slot_elems(g);
    int last_tile = -1;
    for (int item = cta; item < items; item += n_cta) {
      const int tile = item / kParts, part = item % kParts;
      const int ltm = tile / tiles_n, tn = tile - ltm * tiles_n;
      if (tile != last_tile) {
        if (tid < nranks) {
          wait_flag_sys(flags[rank] + (static_cast<size_t>(tid) * tiles_m_local + ltm) * tiles_n + tn, epoch, abort_flag, g);
        }
        epilogue_warps_sync();
        if (*abort_flag != 0u) return;
        last_tile = tile;
      }
      const int row0 = ltm * kBM + part * kRows;
      const int col0 = tn * bn;
      const int ncols = min(bn, g.N - col0);
      const int vec_per_row = ncols / 8;  // 8 bf16 = 16 bytes (N is a multiple of 8)
      const int nvec = kRows * vec_per_row;
      for (int v0 = tid; v0 < nvec; v0 += 128 * U) {
        uint4 x[U][NR];
        size_t off[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + u * 128;
          const int rr = row0 + v / vec_per_row;
          const int cc = col0 + (v % vec_per_row) * 8;
          off[u] = elem_offset(g, rr, cc);
#pragma unroll
          for (int src = 0; src < NR; ++src)
            if (src < nranks && v < nvec) x[u][src] = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(src) * slot_elems(g) + off[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
          const int v = v0 + u * 128;
          if (v >= nvec) continue;
          float acc[8];
#pragma unroll
          for (int src = 0; src < NR; ++src) {
            if (src < nranks) {
              const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&x[u][src]);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const float2 f = __bfloat1622float2(h[k]);
                acc[2 * k] = src == 0 ? f.x : acc[2 * k] + f.x;
                acc[2 * k + 1] = src == 0 ? f.y : acc[2 * k + 1] + f.y;
              }
            }
          }
          uint4 y;
          __nv_bfloat162* o = reinterpret_cast<__nv_bfloat162*>(&y);
#pragma unroll
          for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
          const int rr = row0 + v / vec_per_row;
          const int cc = col0 + (v % vec_per_row) * 8;
          *reinterpret_cast<uint4*>(out + static_cast<size_t>(rr) * ldo + cc) = y;
        }
      }
    }
  }

  // Switch mode.  Items are 32 rows x one tile width of the rows this rank owns, numbered in the order
  // the tiles are finished (every rank walks the tiles column by column, so all partial copies of a tile
  // appear at about the same time and every wave holds rows of every owner).  Whoever has nothing else
  // to do takes the next item from a counter: the communication CTAs from the start, the epilogue warps
  // of a compute CTA once its tiles are done.  An item waits (bounded) for the tile's flag from every
  // rank, then each thread sums 16 bytes of all ranks' copies in the switch (fp32 accumulation, one
  // rounding to bf16) and writes them to the output.  NT threads take part; WHOLE_CTA picks the barrier.
  template <int NT, bool WHOLE_CTA>
  __device__ __forceinline__ void reduce_switch(const GemmArgs& g, uint32_t epoch, int tid, volatile uint32_t* abort_flag) const {
    __shared__ int s_item;
    __shared__ int s_stop;
    const int tiles_n = (g.N + bn - 1) / bn;
    const int tiles_m_local = rows_per_rank / kBM;
    constexpr int kParts = 4, kRows = kBM / kParts;
    constexpr int U = (kRows * (kBN / 8) + NT - 1) / NT;       // 16-byte vectors per thread and item
    const int items = tiles_m_local * tiles_n * kParts;
    const char* mc = mc_stage + static_cast<size_t>(epoch & 1u) * g.M * g.N * sizeof(__nv_bfloat16);
    for (;;) {
      if (tid == 0) s_item = static_cast<int>(atomicAdd(work, 1u));
      if (WHOLE_CTA) __syncthreads(); else epilogue_warps_sync();
      const int item = s_item;
      if (item >= items) break;                                // the same for every thread
      const int tile = item / kParts, part = item - tile * kParts;
      const int tn = tile / tiles_m_local, ltm = tile - tn * tiles_m_local;
      if (tid < nranks) wait_flag_sys(flags[rank] + (static_cast<size_t>(tid) * tiles_m_local + ltm) * tiles_n + tn, epoch, abort_flag, g);
      if (WHOLE_CTA) __syncthreads(); else epilogue_warps_sync();
      if (tid == 0) s_stop = *abort_flag != 0u ? 1 : 0;
      if (WHOLE_CTA) __syncthreads(); else epilogue_warps_sync();  // also: s_item has been read by everyone
      if (s_stop) break;
      const int lrow0 = ltm * kBM + part * kRows;              // within this rank's rows
      const int col0 = tn * bn;
      const int vec_per_row = min(bn, g.N - col0) / 8;
      const int nvec = kRows * vec_per_row;
      uint4 x[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = tid + u * NT;
        if (v < nvec) {
          const int rr = lrow0 + v / vec_per_row, cc = col0 + (v % vec_per_row) * 8;
          const char* src = mc + (static_cast<size_t>(rank * rows_per_rank + rr) * g.N + cc) * sizeof(__nv_bfloat16);
          asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                       : "=r"(x[u].x), "=r"(x[u].y), "=r"(x[u].z), "=r"(x[u].w)
                       : "l"(src)
                       : "memory");
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int v = tid + u * NT;
        if (v < nvec) {
          const int rr = lrow0 + v / vec_per_row, cc = col0 + (v % vec_per_row) * 8;
          *reinterpret_cast<uint4*>(out + static_cast<size_t>(rr) * ldo + cc) = x[u];
        }
      }
    }
  }

  __device__ __forceinline__ void comm_cta(const GemmArgs& g, uint32_t epoch, int /*cta*/, int /*n_comm*/,
                                           volatile uint32_t* abort_flag, uint8_t*, uint32_t) const {
    if (mc_stage != nullptr) reduce_switch<kThreads, true>(g, epoch, static_cast<int>(threadIdx.x), abort_flag);
  }
  __device__ __forceinline__ void last_cta_out(const GemmArgs&, uint32_t) const {}
};

// ------------------------------------------------------------------ all-gather -> GEMM

struct AgEpilogue {
  int rank, nranks;
  int rows_per_rank;                 // M / nranks, a multiple of 128
  int lda;                           // row stride of the gather buffers, elements
  char* xg[kMaxTpRanks];             // every rank's gather buffer [M, K] bf16
  uint32_t* ready[kMaxTpRanks];      // every rank's chunk counters [M / 128]
  uint32_t* bar[kMaxTpRanks];        // every rank's barrier words [n_comm][nranks] (unused since the done words)
  int done_base;                     // ready[r] + done_base + s: rank s has left its call number (value); see last_cta_out
  StoreEpilogue<false> plain;

  int swiglu;                        // 1: the store applies SwiGLU (see store_swiglu); C is [M, N / 2]
  int chunks_per_tile;               // 32-column pieces per tile (tile width / 32)

  __device__ __forceinline__ void store(const GemmArgs& g, uint32_t epoch, int row, int col, const uint32_t (&r)[32],
                                        int chunk, uint8_t* warp_smem, int lane) const {
    if (swiglu) store_swiglu(g, row, col, r, chunk, warp_smem, lane);
    else plain.store(g, epoch, row, col, r, chunk, warp_smem, lane);
  }

  // SwiGLU in the epilogue.  The weight's rows (the GEMM's columns) come interleaved in groups of 16:
  // columns [32k, 32k+16) are gate features 16k.., columns [32k+16, 32k+32) the up features of the
  // same indices, so one 32-column piece of an accumulator row holds both operands of 16 outputs:
  //   act[row, 16k + j] = silu(acc[32k + j]) * acc[32k + 16 + j]        (fp32 math, one rounding)
  // Up to four pieces (64 outputs = 128 bytes per row) are collected in shared memory and leave as
  // whole rows, 8 lanes per row.  The H = (gate | up) matrix never reaches memory: the kernel
  // writes half the bytes and the separate elementwise pass disappears.
  __device__ __forceinline__ void store_swiglu(const GemmArgs& g, int row, int col, const uint32_t (&r)[32], int chunk,
                                               uint8_t* warp_smem, int lane) const {
    if (col >= g.N) return;  // the same for the whole warp (N is a multiple of 32 here)
    const int part = chunk & 3;
    uint8_t* mine = warp_smem + lane * kEpiRowBytes + part * 32;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      uint4 v;
      uint32_t* w = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const int i = 8 * j + 2 * k;
        const float g0 = __uint_as_float(r[i]), g1 = __uint_as_float(r[i + 1]);
        const float u0 = __uint_as_float(r[16 + i]), u1 = __uint_as_float(r[16 + i + 1]);
        __nv_bfloat162 p = __floats2bfloat162_rn(g0 / (1.0f + __expf(-g0)) * u0, g1 / (1.0f + __expf(-g1)) * u1);
        w[k] = *reinterpret_cast<uint32_t*>(&p);
      }
      *reinterpret_cast<uint4*>(mine + j * 16) = v;
    }
    const bool flush = part == 3 || chunk == chunks_per_tile - 1 || col + 32 >= g.N;
    if (!flush) return;
    __syncwarp();
    const int row_base = row - lane;
    const int out_col = (col - part * 32) / 2;       // first output column of the collected pieces
    const int out_cols = (part + 1) * 16;
    __nv_bfloat16* c = static_cast<__nv_bfloat16*>(g.c);
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int rr = it * 4 + (lane >> 3), seg = lane & 7;
      const int grow = row_base + rr;
      if (grow < g.M && seg * 8 < out_cols) {
        const uint4 v = *reinterpret_cast<const uint4*>(warp_smem + rr * kEpiRowBytes + seg * 16);
        *reinterpret_cast<uint4*>(c + static_cast<size_t>(grow) * g.ldc + out_col + seg * 8) = v;
      }
    }
    __syncwarp();
  }
  static constexpr int kWarpSmemBytes = kEpiWarpBytes;
  static constexpr int kSingleStages = kStages;
  static constexpr int kPairStages = 6;
  __device__ __forceinline__ void warp_begin(uint8_t*, int) const {}
  __device__ __forceinline__ void tile_done(const GemmArgs&, uint32_t, int, int, int, int, uint8_t*) const {}
  __device__ __forceinline__ void after_tiles(const GemmArgs&, uint32_t, int, int, int, int, volatile uint32_t*, uint8_t*) const {}

  // The last CTA of the kernel (every tile done, every row of the gather buffer read): tell every peer
  // that this rank's gather buffer is free for the pushes of the next call.
  __device__ __forceinline__ void last_cta_out(const GemmArgs&, uint32_t epoch) const {
    if (nranks <= 1 || ready[rank] == nullptr) return;
    __threadfence_system();
    for (int p = 0; p < nranks; ++p)
      if (p != rank) st_release_sys_u32(ready[p] + done_base + rank, epoch);
  }

  // A communication CTA: wait until every peer has left the previous use of its gather buffer, then
  // push the local shard to every peer with the TMA engine:
  // bulk copies local memory -> shared memory -> peer memory, a ring of row-sized slots, driven by
  // one thread.  Work items are (peer, chunk of 128 rows, quarter of the chunk), dealt round-robin
  // to the communication CTAs in the order the peers will need them; each finished quarter adds
  // one to the peer's counter for that chunk (kAgPartsPerChunk per chunk and call).
  __device__ __forceinline__ void comm_cta(const GemmArgs& g, uint32_t epoch, int cta, int n_comm,
                                           volatile uint32_t* abort_flag, uint8_t* smem, uint32_t smem_base) const {
    __shared__ uint64_t s_full[kAgSlots];
    const int t = threadIdx.x;
    // A peer's gather buffer may be written again once that peer has LEFT its previous call (it reads
    // the rows until then).  Every rank says so when its kernel ends (last_cta_out), so in a steady
    // sequence of calls this wait finds its word already there: the pushes start at once and do not
    // wait for the peers to start their kernels, as a barrier here would (and did).
    (void)cta;
    if (t < nranks && t != rank) wait_flag_sys(ready[rank] + done_base + t, epoch - 1u, abort_flag, g);
    if (t == 0) {
      for (int i = 0; i < kAgSlots; ++i) mbar_init(smem_u32(&s_full[i]), 1);
      fence_barrier_init();
      fence_proxy_async();
    }
    __syncthreads();
    if (*abort_flag != 0u || t != 0) return;
    (void)smem;
    const uint32_t row_bytes = static_cast<uint32_t>(g.K) * 2u;
    int slots = static_cast<int>((kStages * kStageBytes) / row_bytes);
    if (slots > kAgSlots) slots = kAgSlots;
    const int depth = slots / 2;                       // loads run this many rows ahead of the stores
    const int chunks = rows_per_rank / kBM;
    const int rows_per_part = kBM / kAgPartsPerChunk;
    const int items = (nranks - 1) * chunks * kAgPartsPerChunk;
    uint32_t n_loaded = 0;                             // rows whose load has been issued, over all items
    for (int item = cta; item < items; item += n_comm) {
      const int s = item / (chunks * kAgPartsPerChunk) + 1;
      const int c = (item / kAgPartsPerChunk) % chunks;
      const int part = item % kAgPartsPerChunk;
      const int peer = (rank - s + nranks) % nranks;   // the peer that wants this shard soonest first
      const int row0 = rank * rows_per_rank + c * kBM + part * rows_per_part;
      const uint32_t first = n_loaded;
      bool ok = true;
      for (int i = 0; i < rows_per_part + depth && ok; ++i) {
        if (i < rows_per_part) {
          const uint32_t n = first + i, slot = n % slots;
          // the store that last used this slot must have finished reading it
          if (n >= static_cast<uint32_t>(slots)) {
            // with the full ring (16 slots, stores 8 rows behind) that store is the 8th most recent group
            if (slots == kAgSlots) bulk_wait_read<kAgSlots / 2 - 1>();
            else bulk_wait_read<0>();
          }
          const uint32_t full = smem_u32(&s_full[slot]);
          mbar_arrive_expect_tx(full, row_bytes);
          bulk_load(smem_base + slot * row_bytes, xg[rank] + static_cast<size_t>(row0 + i) * lda * 2, row_bytes, full);
          ++n_loaded;
        }
        const int k = i - depth;
        if (k >= 0) {
          const uint32_t n = first + k, slot = n % slots;
          if (!mbar_wait(smem_u32(&s_full[slot]), (n / slots) & 1u, abort_flag, g.wait_budget_ns)) { ok = false; break; }
          bulk_store(xg[peer] + static_cast<size_t>(row0 + k) * lda * 2, smem_base + slot * row_bytes, row_bytes);
          bulk_commit();
        }
      }
      bulk_wait_all();            // the rows of this quarter are written
      if (!ok) return;
      fence_proxy_async_all();    // writes of the async proxy before the release below
      red_release_sys_add(ready[peer] + (row0 / kBM), 1u);
    }
  }
};

namespace {

// What a fused kernel needs of a communicator: parsed from the bytes mncclCommDeviceHandle returns.
struct CommBinding {
  const volatile uint32_t* abort_word = nullptr;
  volatile uint32_t* progress = nullptr;
  uint64_t budget_ns = 2000000000ull;   // without a communicator: two seconds per wait
};

CommBinding bind_comm(const void* handle, size_t bytes) {
  CommBinding b;
  if (handle == nullptr || bytes < sizeof(CommDev)) return b;
  CommDev d;
  memcpy(&d, handle, sizeof(d));
  b.abort_word = d.abort_word;
  b.progress = d.host_progress;
  if (d.spin_timeout_ns != 0) b.budget_ns = d.spin_timeout_ns;
  return b;
}

bool check_common(int M, int N, int K, int rank, int nranks, const char* who) {
  if (M <= 0 || N <= 0 || K <= 0 || nranks < 1 || nranks > kMaxTpRanks || rank < 0 || rank >= nranks) {
    fprintf(stderr, "[Mini-NCCL] %s: bad shape or rank\n", who);
    return false;
  }
  if (M % nranks != 0 || (M / nranks) % kBM != 0 || N % 8 != 0 || K % 8 != 0) {
    fprintf(stderr, "[Mini-NCCL] %s: needs M / nranks to be a multiple of %d and N, K multiples of 8\n", who, kBM);
    return false;
  }
  return true;
}

}  // namespace
}  // namespace gemm
}  // namespace mnccl

using namespace mnccl;
using namespace mnccl::gemm;

extern "C" {
#define MNCCL_EXPORT __attribute__((visibility("default")))

// Bytes / words a caller must provide (in symmetric memory, zero-filled once).
MNCCL_EXPORT size_t mncclGemmRsStageBytes(int M, int N, int /*nranks*/) {
  // two halves x nranks sources x (M / nranks / 128) x ceil(N / bn) tiles of 128 x bn bf16, bn <= 256
  return size_t(2) * M * (size_t(N) + kBN) * 2;
}
MNCCL_EXPORT size_t mncclGemmRsFlagWords(int M, int N, int nranks) {
  return size_t(nranks) * (M / nranks / kBM) * ((N + 127) / 128);  // sized for the narrowest tile
}
// chunk counters [M / 128], then one "has left call number ..." word per source rank
MNCCL_EXPORT size_t mncclAgGemmReadyWords(int M) { return size_t(M) / kBM + kMaxTpRanks; }
MNCCL_EXPORT size_t mncclAgGemmBarWords(int nranks, int n_comm) { return size_t(nranks) * n_comm; }

// out[M/nranks, N] (rows of this rank) = sum over ranks of A_r[M, K] * B_r[N, K]^T, bf16.
// stage_peers / flag_peers: the staging / flag buffers of EVERY rank as mapped here
// (Communicator.peer_pointers); state: two zero-initialised device words of this rank.
static int gemm_rs_launch(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldo, int rank,
                          int nranks, void* const* stage_peers, void* const* flag_peers, uint32_t* state,
                          const CommBinding& cb, cudaStream_t stream, const void* mc_stage = nullptr, int n_comm_ctas = 0) {
  if (!A || !B || !out || !stage_peers || !flag_peers || !state) return -1;
  if (!check_common(M, N, K, rank, nranks, "GEMM->reduce-scatter")) return -2;
  if (lda == 0) lda = K;
  if (ldb == 0) ldb = K;
  if (ldo == 0) ldo = N;
  CUtensorMap ta, tb;
  std::string why;
  // CTA pairs need every rank's rows to be whole 256-row tiles (the rasterisation works on pairs of m-tiles)
  const bool sw = mc_stage != nullptr && nranks > 1;
  if (sw && (ldo % 8 != 0 || (reinterpret_cast<uintptr_t>(out) & 15u) != 0)) {
    fprintf(stderr, "[Mini-NCCL] GEMM->reduce-scatter through the switch: needs ldo a multiple of 8 and out 16-byte aligned\n");
    return -2;
  }
  // switch mode: a few CTAs only sum finished tiles (16 unless told otherwise; whole clusters)
  int n_comm = sw ? (n_comm_ctas > 0 ? ((n_comm_ctas + 1) & ~1) : 16) : 0;
  if (n_comm > sm_count() / 2) n_comm = (sm_count() / 2) & ~1;
  const bool pair = ((M / nranks) % (2 * kBM)) == 0 && want_pair(M, N, sm_count() - n_comm) &&
                    2 * max_pairs<RsEpilogue>() >= (sm_count() & ~1);
  const int bn = pair ? kBN : pick_tile_n(M, N, sm_count() - n_comm, false);
  if (!make_tensor_map_bf16(&ta, A, M, K, lda, kBM, kBK, &why) ||
      !make_tensor_map_bf16(&tb, B, N, K, ldb, pair ? kBN / 2 : bn, kBK, &why)) {
    fprintf(stderr, "[Mini-NCCL] GEMM->reduce-scatter: %s\n", why.c_str());
    return -3;
  }
  RsEpilogue epi{};
  epi.rank = rank;
  epi.nranks = nranks;
  epi.rows_per_rank = M / nranks;
  epi.out = static_cast<__nv_bfloat16*>(out);
  epi.ldo = ldo;
  epi.bn = bn;
  {
    static const int tiled_env = [] {
      const char* e = getenv("MINI_NCCL_RS_TILED");
      return (e != nullptr && *e != 0) ? atoi(e) : 0;
    }();
    epi.tiled = tiled_env;
  }
  for (int r = 0; r < nranks; ++r) {
    epi.stage[r] = static_cast<char*>(stage_peers[r]);
    epi.flags[r] = static_cast<uint32_t*>(flag_peers[r]);
  }
  epi.mc_stage = sw ? static_cast<const char*>(mc_stage) : nullptr;
  epi.work = state + 2;
  if (sw) epi.tiled = 0;
  GemmArgs g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.err = error_word();
  g.wait_budget_ns = cb.budget_ns;
  g.comm_abort = cb.abort_word;
  g.comm_progress = cb.progress;
  const int tiles_m_local = epi.rows_per_rank / kBM;
  if (sw) {
    g.group_m = M / kBM;                                     // column by column, the same on every rank
    g.m_tile_rotate = 0;
  } else {
    g.group_m = tiles_m_local;
    g.m_tile_rotate = ((rank + 1) % nranks) * tiles_m_local;  // next rank's rows first, own rows last
  }
  g.epoch_ptr = state;
  g.ticket_ptr = state + 1;
  g.work_ptr = sw ? state + 2 : nullptr;
  const int tiles = (M / kBM) * ((N + bn - 1) / bn);
  cudaError_t e;
  if (pair) {
    const int sms = (sm_count() & ~1) - n_comm;
    const int n_gemm = tiles < sms ? tiles : sms;             // tiles is even: M / kBM is
    if (sw) g.n_gemm_ctas = n_gemm;
    e = launch_pair(ta, tb, g, epi, n_gemm + n_comm, stream);
  } else {
    const int sms = sm_count() - n_comm;
    const int n_gemm = tiles < sms ? tiles : sms;
    if (sw) g.n_gemm_ctas = n_gemm;
    e = launch(ta, tb, g, epi, n_gemm + n_comm, stream, bn);
  }
  return e == cudaSuccess ? 0 : static_cast<int>(e) + 1000;
}

MNCCL_EXPORT int mncclGemmReduceScatterBf16(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb,
                                            int ldo, int rank, int nranks, void* const* stage_peers,
                                            void* const* flag_peers, uint32_t* state, cudaStream_t stream) {
  return gemm_rs_launch(A, B, out, M, N, K, lda, ldb, ldo, rank, nranks, stage_peers, flag_peers, state, CommBinding(), stream);
}

// The same under a communicator's failure model: `comm_handle` are the bytes mncclCommDeviceHandle
// returns.  Every wait on a peer then polls the communicator's abort word and takes its budget from
// MINI_NCCL_WATCHDOG_TIMEOUT_MS; the watchdog times the kernel like a collective; a wait that gives up
// is reported to the communicator, which fails for good (mncclCommGetAsyncError, every later call).
MNCCL_EXPORT int mncclGemmReduceScatterBf16Comm(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb,
                                                int ldo, int rank, int nranks, void* const* stage_peers,
                                                void* const* flag_peers, uint32_t* state, const void* comm_handle,
                                                size_t comm_handle_bytes, cudaStream_t stream) {
  return gemm_rs_launch(A, B, out, M, N, K, lda, ldb, ldo, rank, nranks, stage_peers, flag_peers, state,
                        bind_comm(comm_handle, comm_handle_bytes), stream);
}

// The same with the sum taken in the NVSwitch: `mc_stage` is the multicast address of the staging
// (mncclMemPeerPointers); state needs three zero-initialised words; n_comm_ctas CTAs only sum finished
// tiles (0 = 16).  Partial sums are bf16, the switch adds them in fp32 in ITS order and rounds once, so
// the result may differ from the peer-to-peer kernel's in the last bit.  With mc_stage null or one
// rank this is mncclGemmReduceScatterBf16Comm.
MNCCL_EXPORT int mncclGemmReduceScatterBf16Switch(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb,
                                                  int ldo, int rank, int nranks, void* const* stage_peers,
                                                  void* const* flag_peers, uint32_t* state, const void* mc_stage,
                                                  int n_comm_ctas, const void* comm_handle, size_t comm_handle_bytes,
                                                  cudaStream_t stream) {
  return gemm_rs_launch(A, B, out, M, N, K, lda, ldb, ldo, rank, nranks, stage_peers, flag_peers, state,
                        bind_comm(comm_handle, comm_handle_bytes), stream, mc_stage, n_comm_ctas);
}

// C[M, N] = X[M, K] * B[N, K]^T where X is the row-wise concatenation of every rank's shard.
// xg_peers: the gather buffer [M, K] of EVERY rank as mapped here; this rank's shard must
// already be at rows [rank * M/nranks, ...) of its own buffer.  ready_peers / bar_peers: counter
// and barrier words of every rank; state: two zero-initialised device words of this rank.
// n_comm_ctas CTAs of the grid move data instead of computing (0 = default).
static int ag_gemm_launch(void* const* xg_peers, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                          int rank, int nranks, void* const* ready_peers, void* const* bar_peers, uint32_t* state,
                          int n_comm_ctas, bool swiglu, const CommBinding& cb, cudaStream_t stream) {
  if (!xg_peers || !B || !C || !state) return -1;
  if (!check_common(M, N, K, rank, nranks, "all-gather->GEMM")) return -2;
  if (swiglu && (N % 32 != 0 || (ldc != 0 && ldc % 8 != 0) || (reinterpret_cast<uintptr_t>(C) & 15u) != 0)) {
    fprintf(stderr, "[Mini-NCCL] all-gather->GEMM with SwiGLU: needs N a multiple of 32, ldc a multiple of 8 and C 16-byte aligned\n");
    return -2;
  }
  if (nranks > 1 && (!ready_peers || !bar_peers)) return -1;
  if (K * 2 > kStages * kStageBytes / 4) {
    fprintf(stderr, "[Mini-NCCL] all-gather->GEMM: K too large for the row ring (max %d)\n", kStages * kStageBytes / 8);
    return -2;
  }
  if (lda == 0) lda = K;
  if (ldb == 0) ldb = K;
  if (ldc == 0) ldc = swiglu ? N / 2 : N;
  CUtensorMap ta, tb;
  std::string why;
  // The A operand is this rank's own gather buffer: TMA only ever reads local memory.
  const bool pair = ((M / nranks) % (2 * kBM)) == 0 && want_pair(M, N, sm_count() - (nranks > 1 ? 16 : 0)) &&
                    2 * max_pairs<AgEpilogue>() >= (sm_count() & ~1);
  // (the SwiGLU store collects pairs of 32-column pieces: no 224-wide tiles then)
  const int bn = pair ? kBN : pick_tile_n(M, N, sm_count() - (nranks > 1 ? 16 : 0), !swiglu);
  if (!make_tensor_map_bf16(&ta, xg_peers[rank], M, K, lda, kBM, kBK, &why) ||
      !make_tensor_map_bf16(&tb, B, N, K, ldb, pair ? kBN / 2 : bn, kBK, &why)) {
    fprintf(stderr, "[Mini-NCCL] all-gather->GEMM: %s\n", why.c_str());
    return -3;
  }
  const int sms = pair ? (sm_count() & ~1) : sm_count();
  const int all_tiles = (M / kBM) * ((N + bn - 1) / bn);
  int n_comm = 0;
  if (nranks > 1) {
    if (n_comm_ctas > 0) {
      n_comm = n_comm_ctas;
    } else {
      // The tiles need ceil(tiles / CTAs) waves anyway: give the GEMM just enough CTAs for that
      // number of waves and let the rest move data (at least 16, at most 48).
      const int waves = (all_tiles + (sms - 16) - 1) / (sms - 16);
      const int need = (all_tiles + waves - 1) / waves;
      n_comm = sms - need;
      if (n_comm < 16) n_comm = 16;
      if (n_comm > 48) n_comm = 48;
    }
    if (n_comm > sms / 2) n_comm = sms / 2;
    if (pair) n_comm = (n_comm + 1) & ~1;  // communication CTAs come as whole clusters too
  }
  AgEpilogue epi{};
  epi.rank = rank;
  epi.nranks = nranks;
  epi.rows_per_rank = M / nranks;
  epi.lda = lda;
  epi.swiglu = swiglu ? 1 : 0;
  epi.chunks_per_tile = bn / 32;
  epi.done_base = M / kBM;
  for (int r = 0; r < nranks; ++r) {
    epi.xg[r] = static_cast<char*>(xg_peers[r]);
    epi.ready[r] = nranks > 1 ? static_cast<uint32_t*>(ready_peers[r]) : nullptr;
    epi.bar[r] = nranks > 1 ? static_cast<uint32_t*>(bar_peers[r]) : nullptr;
  }
  GemmArgs g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.c = C;
  g.ldc = ldc;
  g.err = error_word();
  g.wait_budget_ns = cb.budget_ns;
  g.comm_abort = cb.abort_word;
  g.comm_progress = cb.progress;
  const int tiles_m_local = epi.rows_per_rank / kBM;
  g.group_m = tiles_m_local;
  g.m_tile_rotate = rank * tiles_m_local;  // local rows first, then the shards in arrival order
  g.epoch_ptr = state;
  g.ticket_ptr = state + 1;
  if (nranks > 1) {
    g.a_ready = epi.ready[rank];
    g.a_ready_mult = static_cast<uint32_t>(kAgPartsPerChunk);
    g.rows_per_chunk = kBM;
    g.a_local_first = rank * tiles_m_local;
    g.a_local_count = tiles_m_local;
  }
  const int tiles = all_tiles;
  int n_gemm = sms - n_comm;
  if (tiles < n_gemm) n_gemm = tiles;
  g.n_gemm_ctas = n_gemm;
  // Every CTA must be resident at once (communication CTAs wait for peers while GEMM CTAs
  // wait for data): the grid never exceeds one CTA per SM.
  cudaError_t e = pair ? launch_pair(ta, tb, g, epi, n_gemm + n_comm, stream)
                       : launch(ta, tb, g, epi, n_gemm + n_comm, stream, bn);
  return e == cudaSuccess ? 0 : static_cast<int>(e) + 1000;
}

MNCCL_EXPORT int mncclAllGatherGemmBf16(void* const* xg_peers, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                        int ldc, int rank, int nranks, void* const* ready_peers, void* const* bar_peers,
                                        uint32_t* state, int n_comm_ctas, cudaStream_t stream) {
  return ag_gemm_launch(xg_peers, B, C, M, N, K, lda, ldb, ldc, rank, nranks, ready_peers, bar_peers, state, n_comm_ctas, false,
                        CommBinding(), stream);
}

// The same with SwiGLU applied in the epilogue: act[M, N / 2] = silu(gate) * up, where B's rows are
// interleaved in groups of 16 (rows [32k, 32k+16) gate features 16k.., rows [32k+16, 32k+32) the up
// features of the same indices).  N must be a multiple of 32; ldc (0 = N / 2) a multiple of 8.
MNCCL_EXPORT int mncclAllGatherGemmSwiGluBf16(void* const* xg_peers, const void* B, void* act, int M, int N, int K, int lda,
                                              int ldb, int ldc, int rank, int nranks, void* const* ready_peers,
                                              void* const* bar_peers, uint32_t* state, int n_comm_ctas, cudaStream_t stream) {
  return ag_gemm_launch(xg_peers, B, act, M, N, K, lda, ldb, ldc, rank, nranks, ready_peers, bar_peers, state, n_comm_ctas, true,
                        CommBinding(), stream);
}

// all-gather -> GEMM (swiglu = 0) or all-gather -> GEMM with SwiGLU (swiglu = 1) under a communicator's
// failure model; see mncclGemmReduceScatterBf16Comm.
MNCCL_EXPORT int mncclAllGatherGemmBf16Comm(void* const* xg_peers, const void* B, void* C, int M, int N, int K, int lda, int ldb,
                                            int ldc, int rank, int nranks, void* const* ready_peers, void* const* bar_peers,
                                            uint32_t* state, int n_comm_ctas, int swiglu, const void* comm_handle,
                                            size_t comm_handle_bytes, cudaStream_t stream) {
  return ag_gemm_launch(xg_peers, B, C, M, N, K, lda, ldb, ldc, rank, nranks, ready_peers, bar_peers, state, n_comm_ctas,
                        swiglu != 0, bind_comm(comm_handle, comm_handle_bytes), stream);
}

// One thread waits (bounded by budget_ns) for a flag that nothing sets, the way the fused kernels wait
// for a peer, and reports like they do.  abort_first: an abort word is pre-set, so the wait must
// return at once.  status: the GemmAbort code the wait left; words[4]: what reached the stand-in
// progress words {status, detail, started, done}.  Host-made failure for tests: nothing faults.
__global__ void flag_wait_probe(GemmArgs g, uint32_t* flag, uint32_t* out) {
  __shared__ volatile uint32_t s_abort;
  s_abort = 0;
  fused_kernel_started(g);
  const uint64_t t0 = globaltimer_ns();
  wait_flag_sys(flag, 1u, &s_abort, g);
  out[0] = s_abort;
  out[1] = static_cast<uint32_t>((globaltimer_ns() - t0) / 1000ull);
  report_failure(g, s_abort);
}

MNCCL_EXPORT int mncclGemmProbeFlagWait(uint64_t budget_ns, int abort_first, uint32_t* status, uint32_t* waited_us,
                                        uint32_t* words) {
  uint32_t* buf = nullptr;  // [0] flag, [1] abort, [2..3] out, [4..7] err words, [8..15] progress stand-in
  if (cudaMalloc(&buf, 64) != cudaSuccess) return -2;
  cudaMemset(buf, 0, 64);
  if (abort_first) {
    const uint32_t one = 1;
    cudaMemcpy(buf + 1, &one, 4, cudaMemcpyHostToDevice);
  }
  GemmArgs g{};
  g.err = buf + 4;
  g.wait_budget_ns = budget_ns;
  g.comm_abort = buf + 1;
  g.comm_progress = buf + 8;
  flag_wait_probe<<<1, 1>>>(g, buf, buf + 2);
  uint32_t host[16] = {0};
  cudaError_t e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaMemcpy(host, buf, 64, cudaMemcpyDeviceToHost);
  cudaFree(buf);
  if (e != cudaSuccess) return static_cast<int>(e) + 1000;
  if (status) *status = host[2];
  if (waited_us) *waited_us = host[3];
  if (words) {
    words[0] = host[10];  // status
    words[1] = host[11];  // detail
    words[2] = host[12];  // started
    words[3] = host[13];  // done (the probe never finishes an epoch: stays 0)
  }
  return 0;
}

}  // extern "C"
