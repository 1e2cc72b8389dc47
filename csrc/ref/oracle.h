// CPU oracles: the host restatement of every device reduction, used by the
// tests and by the host ring path.  Accumulation order and precision are the
// contract the device kernels follow: operands are combined in rank order
// 0..N-1; fp16 / bf16 / fp32 accumulate in fp32 and round once at the end;
// fp64 accumulates in fp64; integers in their own type; Avg is Sum followed by
// a multiplication with float(1/N) (floating types) or a division by N
// (integers).  The AVX2 verifier mirrors the reference benchmark's check
// (reference: tests/perf_test.cpp:106-134).
#pragma once
#include <cstddef>
#include <cstdint>

#include "core/dtype.h"

namespace mnccl {

// out[i] = finalize( op_r in[r][i] ).  `scale` multiplies floating results
// after the reduction (pass 1.0 for none); for Avg the 1/N factor is applied
// in addition.  in_type/out_type may differ for floating types (fused cast):
// inputs are first rounded to wire_type, as the device kernels do.
void oracle_allreduce(DType in_type, DType wire_type, DType out_type, RedOp op, int nranks,
                      const void* const* inputs, void* out, size_t count, double scale);

inline void oracle_allreduce(DType t, RedOp op, int nranks, const void* const* inputs, void* out,
                             size_t count) {
  oracle_allreduce(t, t, t, op, nranks, inputs, out, count, 1.0);
}

// acc[i] = op(acc[i], in[i]) for one pair of same-type host buffers (ring
// reduction step; Avg behaves as Sum here and is finalised by scale_inplace).
void host_reduce_pair(DType t, RedOp op, void* acc, const void* in, size_t count);
// Avg finalisation for the ring path.
void host_avg_finalize(DType t, void* buf, size_t count, int nranks);

// AVX2 sum of two fp32 arrays (scalar fallback when AVX2 is absent).
void sum_f32_avx2(const float* a, const float* b, float* out, size_t n);
// Returns true when |got[i] - want[i]| <= atol for all i; otherwise writes the
// first offending index.  8-wide AVX2 main loop + scalar tail.
bool verify_f32_avx2(const float* got, const float* want, size_t n, float atol, size_t* first_bad);
// Compare against a constant (the reference benchmark's all-ones check).
bool verify_const_f32_avx2(const float* got, float want, size_t n, float atol, size_t* first_bad);
bool cpu_has_avx2();

}  // namespace mnccl
