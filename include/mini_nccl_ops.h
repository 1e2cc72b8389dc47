/* Tensor-parallel compute entry points of libmini_nccl.so (sm_100a): the tcgen05 bf16 GEMM, its two
 * fusions with a collective, and the elementwise piece between them.  Additions without a
 * counterpart in the reference, whose library ends at ncclAllReduce (include/mini_nccl_api.h:52-69
 * there).  C linkage; every call is asynchronous on `stream`; return value 0 = launched, < 0 = bad
 * arguments (-1 null / empty, -2 shape or alignment, -3 tensor map), >= 1000 = cudaError_t + 1000.
 *
 * Conventions: matrices are row-major with the K (inner) dimension contiguous, "ld" arguments are row
 * strides in ELEMENTS (0 = dense), operands are bf16, accumulation is fp32.
 *   C[M, N] = A[M, K] * B[N, K]^T          (B is a weight matrix in nn.Linear layout)
 * Operand pointers must be 16-byte aligned and lda / ldb multiples of 8.
 */
#ifndef MINI_NCCL_OPS_H_
#define MINI_NCCL_OPS_H_

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- GEMM alone ------------------------------------------------------------------------------- */

/* out_f32 = 0: C is bf16; 1: C is fp32. */
int mncclGemmBf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc, int out_f32,
                  cudaStream_t stream);

/* First failed (bounded) wait of any GEMM kernel launched so far on the current device: 0 = none.
 * Synchronises the device, reads the word, clears it.  Returns 0, or a negative code. */
int mncclGemmStatus(uint32_t* status);

/* Kernel choice for the calls that follow: -1 automatic, 0 single-CTA 128 x {256,224,192,128} tiles,
 * 1 CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles).  Initial value from MINI_NCCL_GEMM_PAIR. */
void mncclGemmSetPairMode(int mode);

/* The host-side choice for an M x N product on `ctas` CTAs, without a launch (needs no GPU). */
void mncclGemmPlan(int M, int N, int ctas, int narrow, int* tile_n, int* pair);

/* The tiles worker `worker` of `n_workers` (CTAs, or CTA pairs with pair = 1) visits, in the kernels'
 * own order, as (tm, tn) in 128-row tiles; host arithmetic only.  Returns the number of tiles. */
int mncclGemmTileOrder(int M, int N, int bn, int group_m, int rotate, int pair, int n_workers, int worker, int* out_tm,
                       int* out_tn, int max);

/* CTA pairs of the pair kernel that the current device holds at once. */
int mncclGemmMaxPairs(void);

/* ---- GEMM -> reduce-scatter ---------------------------------------------------------------------
 * Every rank multiplies its K-slice, P_r = A_r[M, K_r] * B_r[N, K_r]^T; out[M / nranks, N] on rank i
 * receives rows [i * M / nranks, ...) of the sum over ranks, added in rank order in fp32.
 * Workspaces (symmetric memory from mncclMemAlloc, zero-filled once, same size on every rank):
 *   staging  mncclGemmRsStageBytes(M, N, nranks) bytes,
 *   flags    mncclGemmRsFlagWords(M, N, nranks) 32-bit words;
 * stage_peers / flag_peers are those buffers of EVERY rank as mapped here (mncclMemPeerPointers);
 * state: two zero-initialised 32-bit device words of this rank (call counter and exit ticket),
 * kept between calls and never touched by the caller.
 * Needs M / nranks to be a multiple of 128 and N, K_r multiples of 8.  One rank runs locally. */
size_t mncclGemmRsStageBytes(int M, int N, int nranks);
size_t mncclGemmRsFlagWords(int M, int N, int nranks);
int mncclGemmReduceScatterBf16(const void* A, const void* B, void* out, int M, int N, int K, int lda, int ldb, int ldo,
                               int rank, int nranks, void* const* stage_peers, void* const* flag_peers, uint32_t* state,
                               cudaStream_t stream);

/* ---- all-gather -> GEMM -------------------------------------------------------------------------
 * X[M, K] is sharded by rows; C[M, N_r] = X * B_r[N_r, K]^T on every rank.  xg_peers: the gather
 * buffer [M, K] (symmetric memory) of EVERY rank as mapped here; before the call this rank's shard
 * must sit at rows [rank * M / nranks, ...) of its own buffer.  ready_peers / bar_peers: counter and
 * barrier words of every rank (mncclAgGemmReadyWords(M) / mncclAgGemmBarWords(nranks, n_comm) words,
 * zero-filled once; with n_comm_ctas = 0 size the barrier words for n_comm = 74, which covers every
 * automatic choice); state as above.  n_comm_ctas CTAs of the grid move data instead of computing
 * (0 = chosen from the shape).  K is at most 24576.  TMA only reads local memory: peers push their
 * shards. */
size_t mncclAgGemmReadyWords(int M);
size_t mncclAgGemmBarWords(int nranks, int n_comm);
int mncclAllGatherGemmBf16(void* const* xg_peers, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                           int rank, int nranks, void* const* ready_peers, void* const* bar_peers, uint32_t* state,
                           int n_comm_ctas, cudaStream_t stream);

/* ---- SwiGLU ---------------------------------------------------------------------------------------
 * act[M, F] = silu(h[:, 0:F]) * h[:, F:2F], bf16 in and out, fp32 math, one rounding.
 * F, ldh, lda multiples of 8; both pointers 16-byte aligned. */
int mncclSwiGluBf16(const void* h, void* act, int M, int F, long ldh, long lda, cudaStream_t stream);

#ifdef __cplusplus
}
#endif

#endif /* MINI_NCCL_OPS_H_ */
