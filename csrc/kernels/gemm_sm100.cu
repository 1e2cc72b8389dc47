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
#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include "kernels/gemm2_kernel.cuh"
#include "mem/cuda_driver.h"

namespace mnccl {
namespace gemm {

// -------------------------------------------------------------------- host

namespace {

std::mutex g_mu;
// -1: automatic, 0: single-CTA kernel, 1: CTA-pair kernel; MINI_NCCL_GEMM_PAIR sets the initial value
int pair_mode_from_env() {
  const char* e = getenv("MINI_NCCL_GEMM_PAIR");
  if (e == nullptr || *e == 0) return -1;
  const int v = atoi(e);
  return v < 0 ? -1 : (v > 0 ? 1 : 0);
}
int g_use_pair = pair_mode_from_env();
uint32_t* g_err_dev[kMaxDevices] = {};  // one error word per device of the process
float* g_split_ws[kMaxDevices] = {};    // split-K workspace per device (fp32 partial tiles), allocated on first use
uint32_t* g_split_cnt[kMaxDevices] = {};
constexpr int kSplitMaxItems = 80;      // K-slices in flight: at most one per CTA pair

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
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  if (g_err_dev[dev] == nullptr) {
    uint32_t* p = nullptr;
    if (cudaMalloc(&p, 64) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, 64);
    g_err_dev[dev] = p;
  }
  return g_err_dev[dev];
}

// Workspace of the split last wave: kSplitMaxItems partial tiles of 256 x 256 fp32 (20 MB) and one
// counter per 32-row quarter.  Allocated once per device, the first time a shape is split (not under
// stream capture: call the GEMM once before capturing).  Null when the allocation fails: no split then.
bool split_workspace(float** ws, uint32_t** cnt) {
  std::lock_guard<std::mutex> lk(g_mu);
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= kMaxDevices) dev = 0;
  if (g_split_ws[dev] == nullptr) {
    float* w = nullptr;
    uint32_t* c = nullptr;
    if (cudaMalloc(&w, size_t(kSplitMaxItems) * 256 * 256 * 4) != cudaSuccess ||
        cudaMalloc(&c, size_t(kSplitMaxItems) * 8 * 4) != cudaSuccess) {
      (void)cudaGetLastError();
      if (w) cudaFree(w);
      return false;
    }
    cudaMemset(c, 0, size_t(kSplitMaxItems) * 8 * 4);
    g_split_ws[dev] = w;
    g_split_cnt[dev] = c;
  }
  *ws = g_split_ws[dev];
  *cnt = g_split_cnt[dev];
  return true;
}

// Split-K plan of the CTA-pair kernel: tiles2 tiles on n_pairs pairs, num_kb k-blocks per tile.  When
// the last wave holds at most half as many tiles as there are pairs, each of its tiles is cut into at
// most 8 slices of at least 4 k-blocks so that all slices still form ONE wave (their warps wait for one
// another, which is only safe because they are all resident at the same time).  Returns false for "no split".
bool plan_split(int tiles2, int n_pairs, int num_kb, int* first, int* s, int* kb) {
  const char* e = getenv("MINI_NCCL_GEMM_SPLIT_K");
  if (e != nullptr && *e == '0') return false;
  if (n_pairs < 2 || tiles2 <= n_pairs) return false;        // a single wave: nothing to balance
  const int rem = tiles2 % n_pairs;
  if (rem == 0 || 2 * rem > n_pairs) return false;
  int slices = n_pairs / rem;
  if (slices > kBN / 32) slices = kBN / 32;                     // a slice's warp sums whole 32-column pieces
  if (slices > num_kb / 4) slices = num_kb / 4;
  if (slices * rem > kSplitMaxItems) slices = kSplitMaxItems / rem;
  if (slices < 2) return false;
  const int per = (num_kb + slices - 1) / slices;
  *first = tiles2 - rem;
  *kb = per;
  *s = (num_kb + per - 1) / per;                                // no empty slice
  if (*s < 2) return false;
  // Measured on B200: a 256 x 256 pair tile takes about 3 us + 0.33 us per k-block, and cutting it costs
  // about 7 us (partial sums to the workspace, the meeting of the slices, the sum): 4096 x 3584 x 4096
  // gains 12 us with 8 slices, 4096 x 4096 x 1792 loses 1 us with 2, 4096 x 4096 x 512 loses 4 us.
  const long tile_ns = 3000 + 330L * num_kb;
  return tile_ns * (*s - 1) / *s > 9000;
}

int pick_tile_n(int M, int N, int ctas, bool allow_224) {
  const int cand[4] = {256, 224, 192, 128};  // 128: small products that leave most SMs without a tile
  int best = 256;
  long best_cost = -1;
  const int tiles_m = (M + kBM - 1) / kBM;
  for (int i = 0; i < 4; ++i) {
    const int bn = cand[i];
    if ((bn == 224 || bn == 128) && !allow_224) continue;
    const long tiles = static_cast<long>(tiles_m) * ((N + bn - 1) / bn);
    const long waves = (tiles + ctas - 1) / ctas;
    // Measured on B200 (4096 x 4096 x 1792): a wave of 256-wide tiles takes 13.9 us, of 192-wide
    // tiles 12.2 us: the time per tile is about a + b * bn with a / b ~ 256 columns, so a narrower
    // tile only pays when it removes a whole wave.
    const long cost = waves * (bn + 256);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best = bn;
    }
  }
  return best;
}

bool want_pair(int M, int N, int ctas) {
  if (g_use_pair == 0 || M < 2 * kBM || N < kBN || ctas < 2) return false;
  if (g_use_pair == 1) return true;
  // Measured on B200: pairs win by 5-15 % (a third less operand traffic from L2 per FLOP) once
  // they have enough tiles; with far fewer tiles than pairs, or a worse last wave, single tiles win.
  const long pairs = ctas / 2;
  const long t2 = static_cast<long>((M + 2 * kBM - 1) / (2 * kBM)) * ((N + kBN - 1) / kBN);
  const long t1 = static_cast<long>((M + kBM - 1) / kBM) * ((N + kBN - 1) / kBN);
  if (2 * t2 < pairs) return false;  // small products: narrower single-CTA tiles reach more SMs
  const double fill2 = static_cast<double>(t2) / static_cast<double>(((t2 + pairs - 1) / pairs) * pairs);
  const double fill1 = static_cast<double>(t1) / static_cast<double>(((t1 + ctas - 1) / ctas) * ctas);
  return fill2 >= fill1 - 0.04;
}

int pair_mode() { return g_use_pair; }
void set_pair_mode(int m) { g_use_pair = m; }

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
  GemmArgs g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.c = C;
  g.ldc = ldc;
  g.err = error_word();
  g.wait_budget_ns = 2000000000ull;
  g.group_m = 8;
  cudaError_t e;
  const bool pair = want_pair(M, N, sm_count());
  if (pair) {
    // CTA pairs: 256 x 256 tiles, each CTA loads 128 rows of A and 128 rows (half of N) of B
    if (!make_tensor_map_bf16(&ta, A, M, K, lda, kBM, kBK, &why) || !make_tensor_map_bf16(&tb, B, N, K, ldb, kBN / 2, kBK, &why)) {
      fprintf(stderr, "[Mini-NCCL] GEMM: %s\n", why.c_str());
      return -3;
    }
    const int tiles2 = ((M + 2 * kBM - 1) / (2 * kBM)) * ((N + kBN - 1) / kBN);
    int grid = 2 * tiles2;
    if (grid > (sm_count() & ~1)) grid = sm_count() & ~1;
    const int pairs = std::min(grid / 2, max_pairs<StoreEpilogue<false>>());
    int first = 0, slices = 0, per = 0;
    if (plan_split(tiles2, pairs, (K + kBK - 1) / kBK, &first, &slices, &per) && split_workspace(&g.split_ws, &g.split_cnt)) {
      g.split_first = first;
      g.split_s = slices;
      g.split_kb = per;
    }
    e = out_f32 ? launch_pair(ta, tb, g, StoreEpilogue<true>{}, grid, stream) : launch_pair(ta, tb, g, StoreEpilogue<false>{}, grid, stream);
  } else {
    const int bn = pick_tile_n(M, N, sm_count(), true);
    if (!make_tensor_map_bf16(&ta, A, M, K, lda, kBM, kBK, &why) || !make_tensor_map_bf16(&tb, B, N, K, ldb, bn, kBK, &why)) {
      fprintf(stderr, "[Mini-NCCL] GEMM: %s\n", why.c_str());
      return -3;
    }
    const int tiles = ((M + kBM - 1) / kBM) * ((N + bn - 1) / bn);
    const int grid = tiles < sm_count() ? tiles : sm_count();
    e = out_f32 ? launch(ta, tb, g, StoreEpilogue<true>{}, grid, stream, bn) : launch(ta, tb, g, StoreEpilogue<false>{}, grid, stream, bn);
  }
  return e == cudaSuccess ? 0 : static_cast<int>(e) + 1000;
}

// Pairs of CTAs (clusters of 2) of the GEMM kernel that fit the current device at once.
MNCCL_EXPORT int mncclGemmMaxPairs(void) { return max_pairs<StoreEpilogue<false>>(); }

// Kernel choice for the calls that follow: -1 automatic, 0 single-CTA tiles, 1 CTA pairs (cta_group::2).
MNCCL_EXPORT void mncclGemmSetPairMode(int mode) { set_pair_mode(mode); }

// The host-side choice for an M x N product on `ctas` CTAs, without launching anything (needs no
// GPU): *tile_n = tile width of the single-CTA kernel (`narrow` = 1 admits 224 and 128), *pair = 1
// when the CTA-pair kernel would be taken instead.
MNCCL_EXPORT void mncclGemmPlan(int M, int N, int ctas, int narrow, int* tile_n, int* pair) {
  if (tile_n) *tile_n = pick_tile_n(M, N, ctas, narrow != 0);
  if (pair) *pair = want_pair(M, N, ctas) ? 1 : 0;
}

// The split-K plan of the CTA-pair kernel for an M x N x K product on `pairs` CTA pairs, without launching
// anything (needs no GPU): returns 1 and the first split work item, the slices per tile and the k-blocks
// per slice when the last, partial wave is cut along K, else 0.
MNCCL_EXPORT int mncclGemmSplitPlan(int M, int N, int K, int pairs, int* first, int* slices, int* kb_per_slice) {
  if (M <= 0 || N <= 0 || K <= 0 || pairs <= 0) return 0;
  const int tiles2 = ((M + 2 * kBM - 1) / (2 * kBM)) * ((N + kBN - 1) / kBN);
  int f = 0, s = 0, k = 0;
  if (!plan_split(tiles2, pairs, (K + kBK - 1) / kBK, &f, &s, &k)) return 0;
  if (first) *first = f;
  if (slices) *slices = s;
  if (kb_per_slice) *kb_per_slice = k;
  return 1;
}

// The tiles worker `worker` of `n_workers` visits, in order, exactly as the kernels walk them (host
// arithmetic only, for tests): single-CTA kernel: worker = CTA, tiles of 128 x bn; pair kernel
// (`pair` = 1): worker = CTA pair, 256 x 256 tiles, reported as the two 128-row tiles (tm, tm + 1)
// of its CTAs.  group_m / rotate are the values the entry points put into GemmArgs (in 128-row
// tiles).  Writes up to `max` (tm, tn) pairs; returns the number of 128-row tiles visited.
MNCCL_EXPORT int mncclGemmTileOrder(int M, int N, int bn, int group_m, int rotate, int pair, int n_workers, int worker,
                                    int* out_tm, int* out_tn, int max) {
  if (M <= 0 || N <= 0 || bn <= 0 || n_workers <= 0 || worker < 0 || worker >= n_workers) return -1;
  GemmArgs g{};
  g.M = M;
  g.N = N;
  int n = 0;
  if (pair) {
    g.group_m = group_m > 1 ? group_m / 2 : 1;          // as gemm2_bf16_kernel derives them
    g.m_tile_rotate = rotate / 2;
    const int tiles_m2 = (M + 2 * kBM - 1) / (2 * kBM), tiles_n = (N + kBN - 1) / kBN;
    for (int t = worker; t < tiles_m2 * tiles_n; t += n_workers) {
      int tm2, tn;
      tile_coords(g, t, tiles_m2, tiles_n, &tm2, &tn);
      for (int cta = 0; cta < 2; ++cta, ++n)
        if (n < max) { out_tm[n] = tm2 * 2 + cta; out_tn[n] = tn; }
    }
  } else {
    g.group_m = group_m;
    g.m_tile_rotate = rotate;
    const int tiles_m = (M + kBM - 1) / kBM, tiles_n = (N + bn - 1) / bn;
    for (int t = worker; t < tiles_m * tiles_n; t += n_workers, ++n) {
      int tm, tn;
      tile_coords(g, t, tiles_m, tiles_n, &tm, &tn);
      if (n < max) { out_tm[n] = tm; out_tn[n] = tn; }
    }
  }
  return n;
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
