// Exported C entry points of the host oracle (csrc/ref/oracle.h): the rank-ordered restatement of
// the device arithmetic and the AVX2 verifier, for bindings (mini_nccl_b200/utils/oracle.py), the
// benchmark's correctness battery and C users.  The reference verifies with AVX2 inside its
// benchmark only (reference: tests/perf_test.cpp:102-134).
#include <cstddef>
#include <cstdint>
#include <exception>

#include "core/dtype.h"
#include "core/error.h"
#include "ref/oracle.h"

using namespace mnccl;

namespace {
template <typename Fn>
int guarded(Fn&& fn) {
  try {
    return fn();
  } catch (const Error& e) {
    return 100 + static_cast<int>(e.code());
  } catch (const std::exception&) {
    return 99;
  }
}
}  // namespace

extern "C" {
#define MNCCL_EXPORT __attribute__((visibility("default")))

MNCCL_EXPORT int mnccl_oracle_allreduce(int in_t, int wire_t, int out_t, int op, int nranks, const void* const* inputs,
                                        void* out, size_t count, double scale) {
  return guarded([&] {
    oracle_allreduce(static_cast<DType>(in_t), static_cast<DType>(wire_t), static_cast<DType>(out_t),
                     static_cast<RedOp>(op), nranks, inputs, out, count, scale);
    return 0;
  });
}
MNCCL_EXPORT int mnccl_verify_f32(const float* got, const float* want, size_t n, float atol, size_t* first_bad) {
  return verify_f32_avx2(got, want, n, atol, first_bad) ? 0 : 1;
}
MNCCL_EXPORT int mnccl_verify_const_f32(const float* got, float want, size_t n, float atol, size_t* first_bad) {
  return verify_const_f32_avx2(got, want, n, atol, first_bad) ? 0 : 1;
}
MNCCL_EXPORT void mnccl_sum_f32(const float* a, const float* b, float* out, size_t n) { sum_f32_avx2(a, b, out, n); }
MNCCL_EXPORT int mnccl_cpu_has_avx2() { return cpu_has_avx2() ? 1 : 0; }
MNCCL_EXPORT uint16_t mnccl_float_to_bf16(float f) { return float_to_bf16(f); }
MNCCL_EXPORT uint16_t mnccl_float_to_half(float f) { return float_to_half(f); }
MNCCL_EXPORT float mnccl_bf16_to_float(uint16_t h) { return bf16_to_float(h); }
MNCCL_EXPORT float mnccl_half_to_float(uint16_t h) { return half_to_float(h); }

}  // extern "C"
