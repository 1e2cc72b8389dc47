#include "ref/oracle.h"

#include <algorithm>
#include <cmath>
#include <immintrin.h>
#include <type_traits>

#include "core/error.h"

namespace mnccl {
namespace {

template <typename A>
inline A apply(RedOp op, A a, A b) {
  switch (op) {
    case RedOp::Sum: case RedOp::Avg: return a + b;
    case RedOp::Prod: return a * b;
    case RedOp::Max: return a > b ? a : b;
    case RedOp::Min: return a < b ? a : b;
  }
  return a;
}

inline float load_as_float(DType t, const void* p, size_t i) {
  switch (t) {
    case DType::Float32: return static_cast<const float*>(p)[i];
    case DType::Float16: return half_to_float(static_cast<const uint16_t*>(p)[i]);
    case DType::Bfloat16: return bf16_to_float(static_cast<const uint16_t*>(p)[i]);
    default: return 0.f;
  }
}
inline void store_from_float(DType t, void* p, size_t i, float v) {
  switch (t) {
    case DType::Float32: static_cast<float*>(p)[i] = v; break;
    case DType::Float16: static_cast<uint16_t*>(p)[i] = float_to_half(v); break;
    case DType::Bfloat16: static_cast<uint16_t*>(p)[i] = float_to_bf16(v); break;
    default: break;
  }
}
inline float round_to(DType t, float v) {
  switch (t) {
    case DType::Float16: return half_to_float(float_to_half(v));
    case DType::Bfloat16: return bf16_to_float(float_to_bf16(v));
    default: return v;
  }
}
inline bool is_f32_family(DType t) {
  return t == DType::Float32 || t == DType::Float16 || t == DType::Bfloat16;
}

template <typename T>
void int_allreduce(RedOp op, int n, const void* const* in, void* out, size_t count) {
  T* o = static_cast<T*>(out);
  for (size_t i = 0; i < count; ++i) {
    T acc = static_cast<const T*>(in[0])[i];
    for (int r = 1; r < n; ++r) {
      T v = static_cast<const T*>(in[r])[i];
      if (op == RedOp::Sum || op == RedOp::Avg) {
        // Wrap-around arithmetic, as the device does (avoid signed-overflow UB).
        using U = typename std::make_unsigned<T>::type;
        acc = static_cast<T>(static_cast<U>(acc) + static_cast<U>(v));
      } else if (op == RedOp::Prod) {
        using U = typename std::make_unsigned<T>::type;
        acc = static_cast<T>(static_cast<U>(acc) * static_cast<U>(v));
      } else {
        acc = apply<T>(op, acc, v);
      }
    }
    if (op == RedOp::Avg) acc = static_cast<T>(acc / static_cast<T>(n));
    o[i] = acc;
  }
}

template <typename T>
void int_pair(RedOp op, void* acc_, const void* in_, size_t count) {
  T* a = static_cast<T*>(acc_);
  const T* b = static_cast<const T*>(in_);
  using U = typename std::make_unsigned<T>::type;
  for (size_t i = 0; i < count; ++i) {
    if (op == RedOp::Sum || op == RedOp::Avg) a[i] = static_cast<T>(static_cast<U>(a[i]) + static_cast<U>(b[i]));
    else if (op == RedOp::Prod) a[i] = static_cast<T>(static_cast<U>(a[i]) * static_cast<U>(b[i]));
    else a[i] = apply<T>(op, a[i], b[i]);
  }
}

}  // namespace

void oracle_allreduce(DType in_type, DType wire_type, DType out_type, RedOp op, int nranks,
                      const void* const* inputs, void* out, size_t count, double scale) {
  if (nranks <= 0) fail(Result::InvalidArgument, "oracle: nranks must be positive");
  if (is_f32_family(in_type)) {
    if (!is_f32_family(wire_type) || !is_f32_family(out_type))
      fail(Result::InvalidArgument, "oracle: mixed float/int cast");
    // One factor, computed in double and rounded once, exactly as the launch
    // code computes CollArgs::scale_f.
    const float post = static_cast<float>(scale * (op == RedOp::Avg ? 1.0 / static_cast<double>(nranks) : 1.0));
    for (size_t i = 0; i < count; ++i) {
      float acc = round_to(wire_type, load_as_float(in_type, inputs[0], i));
      for (int r = 1; r < nranks; ++r)
        acc = apply<float>(op, acc, round_to(wire_type, load_as_float(in_type, inputs[r], i)));
      if (post != 1.0f) acc = acc * post;
      store_from_float(out_type, out, i, acc);
    }
    return;
  }
  if (in_type != wire_type || in_type != out_type) fail(Result::InvalidArgument, "oracle: cast only between floating types");
  switch (in_type) {
    case DType::Float64: {
      double* o = static_cast<double*>(out);
      for (size_t i = 0; i < count; ++i) {
        double acc = static_cast<const double*>(inputs[0])[i];
        for (int r = 1; r < nranks; ++r) acc = apply<double>(op, acc, static_cast<const double*>(inputs[r])[i]);
        const double post = scale * (op == RedOp::Avg ? 1.0 / static_cast<double>(nranks) : 1.0);
        if (post != 1.0) acc = acc * post;
        o[i] = acc;
      }
      break;
    }
    case DType::Int8: int_allreduce<int8_t>(op, nranks, inputs, out, count); break;
    case DType::Uint8: int_allreduce<uint8_t>(op, nranks, inputs, out, count); break;
    case DType::Int32: int_allreduce<int32_t>(op, nranks, inputs, out, count); break;
    case DType::Uint32: int_allreduce<uint32_t>(op, nranks, inputs, out, count); break;
    case DType::Int64: int_allreduce<int64_t>(op, nranks, inputs, out, count); break;
    case DType::Uint64: int_allreduce<uint64_t>(op, nranks, inputs, out, count); break;
    default: fail(Result::InvalidArgument, "oracle: bad dtype");
  }
}

void host_reduce_pair(DType t, RedOp op, void* acc, const void* in, size_t count) {
  switch (t) {
    case DType::Float32: {
      float* a = static_cast<float*>(acc);
      const float* b = static_cast<const float*>(in);
      if (op == RedOp::Sum || op == RedOp::Avg) { sum_f32_avx2(a, b, a, count); break; }
      for (size_t i = 0; i < count; ++i) a[i] = apply<float>(op, a[i], b[i]);
      break;
    }
    case DType::Float64: {
      double* a = static_cast<double*>(acc);
      const double* b = static_cast<const double*>(in);
      for (size_t i = 0; i < count; ++i) a[i] = apply<double>(op, a[i], b[i]);
      break;
    }
    case DType::Float16: case DType::Bfloat16: {
      uint16_t* a = static_cast<uint16_t*>(acc);
      const uint16_t* b = static_cast<const uint16_t*>(in);
      for (size_t i = 0; i < count; ++i) {
        float x = t == DType::Float16 ? half_to_float(a[i]) : bf16_to_float(a[i]);
        float y = t == DType::Float16 ? half_to_float(b[i]) : bf16_to_float(b[i]);
        float r = apply<float>(op, x, y);
        a[i] = t == DType::Float16 ? float_to_half(r) : float_to_bf16(r);
      }
      break;
    }
    case DType::Int8: int_pair<int8_t>(op, acc, in, count); break;
    case DType::Uint8: int_pair<uint8_t>(op, acc, in, count); break;
    case DType::Int32: int_pair<int32_t>(op, acc, in, count); break;
    case DType::Uint32: int_pair<uint32_t>(op, acc, in, count); break;
    case DType::Int64: int_pair<int64_t>(op, acc, in, count); break;
    case DType::Uint64: int_pair<uint64_t>(op, acc, in, count); break;
  }
}

void host_avg_finalize(DType t, void* buf, size_t count, int n) {
  switch (t) {
    case DType::Float32: { float s = static_cast<float>(1.0 / n); float* p = static_cast<float*>(buf); for (size_t i = 0; i < count; ++i) p[i] *= s; break; }
    case DType::Float64: { double s = 1.0 / n; double* p = static_cast<double*>(buf); for (size_t i = 0; i < count; ++i) p[i] *= s; break; }
    case DType::Float16: { float s = static_cast<float>(1.0 / n); uint16_t* p = static_cast<uint16_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] = float_to_half(half_to_float(p[i]) * s); break; }
    case DType::Bfloat16: { float s = static_cast<float>(1.0 / n); uint16_t* p = static_cast<uint16_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] = float_to_bf16(bf16_to_float(p[i]) * s); break; }
    case DType::Int8: { int8_t* p = static_cast<int8_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] = static_cast<int8_t>(p[i] / n); break; }
    case DType::Uint8: { uint8_t* p = static_cast<uint8_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] = static_cast<uint8_t>(p[i] / n); break; }
    case DType::Int32: { int32_t* p = static_cast<int32_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] /= n; break; }
    case DType::Uint32: { uint32_t* p = static_cast<uint32_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] /= static_cast<uint32_t>(n); break; }
    case DType::Int64: { int64_t* p = static_cast<int64_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] /= n; break; }
    case DType::Uint64: { uint64_t* p = static_cast<uint64_t*>(buf); for (size_t i = 0; i < count; ++i) p[i] /= static_cast<uint64_t>(n); break; }
  }
}

bool cpu_has_avx2() {
  static const bool has = __builtin_cpu_supports("avx2");
  return has;
}

namespace {
__attribute__((target("avx2"))) void sum_avx2_impl(const float* a, const float* b, float* out, size_t n) {
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m256 x = _mm256_loadu_ps(a + i);
    __m256 y = _mm256_loadu_ps(b + i);
    _mm256_storeu_ps(out + i, _mm256_add_ps(x, y));
  }
  for (; i < n; ++i) out[i] = a[i] + b[i];
}

__attribute__((target("avx2"))) bool verify_avx2_impl(const float* got, const float* want, float want_const,
                                                      bool use_const, size_t n, float atol, size_t* bad) {
  const __m256 tol = _mm256_set1_ps(atol);
  const __m256 absmask = _mm256_castsi256_ps(_mm256_set1_epi32(0x7fffffff));
  const __m256 cvec = _mm256_set1_ps(want_const);
  size_t i = 0;
  for (; i + 8 <= n; i += 8) {
    __m256 g = _mm256_loadu_ps(got + i);
    __m256 w = use_const ? cvec : _mm256_loadu_ps(want + i);
    __m256 d = _mm256_and_ps(_mm256_sub_ps(g, w), absmask);
    // NLE also flags NaN differences (unordered compares true).
    int mask = _mm256_movemask_ps(_mm256_cmp_ps(d, tol, _CMP_NLE_UQ));
    if (mask) {
      if (bad) *bad = i + static_cast<size_t>(__builtin_ctz(static_cast<unsigned>(mask)));
      return false;
    }
  }
  for (; i < n; ++i) {
    float w = use_const ? want_const : want[i];
    if (!(std::fabs(got[i] - w) <= atol)) {
      if (bad) *bad = i;
      return false;
    }
  }
  return true;
}
}  // namespace

void sum_f32_avx2(const float* a, const float* b, float* out, size_t n) {
  if (cpu_has_avx2()) return sum_avx2_impl(a, b, out, n);
  for (size_t i = 0; i < n; ++i) out[i] = a[i] + b[i];
}

static bool verify_scalar(const float* got, const float* want, float c, bool use_const, size_t n, float atol, size_t* bad) {
  for (size_t i = 0; i < n; ++i) {
    float w = use_const ? c : want[i];
    if (!(std::fabs(got[i] - w) <= atol)) {
      if (bad) *bad = i;
      return false;
    }
  }
  return true;
}

bool verify_f32_avx2(const float* got, const float* want, size_t n, float atol, size_t* first_bad) {
  if (cpu_has_avx2()) return verify_avx2_impl(got, want, 0.f, false, n, atol, first_bad);
  return verify_scalar(got, want, 0.f, false, n, atol, first_bad);
}

bool verify_const_f32_avx2(const float* got, float want, size_t n, float atol, size_t* first_bad) {
  if (cpu_has_avx2()) return verify_avx2_impl(got, nullptr, want, true, n, atol, first_bad);
  return verify_scalar(got, nullptr, want, true, n, atol, first_bad);
}

}  // namespace mnccl
