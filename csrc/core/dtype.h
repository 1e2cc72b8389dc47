// Data types and reduction operators shared by host code (oracle, host ring
// reduction) and the launch wrappers.  Numeric values equal ncclDataType_t /
// ncclRedOp_t (reference: include/mini_nccl_api.h:29-49).  The reference
// implements only fp32 / fp64 / int32 with Sum / Prod / Max / Min (reference:
// src/api.cpp:101-128); all ten types and Avg are implemented here.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cstring>

namespace mnccl {

enum class DType : int {
  Int8 = 0, Uint8 = 1, Int32 = 2, Uint32 = 3, Int64 = 4, Uint64 = 5,
  Float16 = 6, Float32 = 7, Float64 = 8, Bfloat16 = 9
};
constexpr int kNumDTypes = 10;

enum class RedOp : int { Sum = 0, Prod = 1, Max = 2, Min = 3, Avg = 4 };
constexpr int kNumRedOps = 5;

inline bool valid_dtype(int d) { return d >= 0 && d < kNumDTypes; }
inline bool valid_op(int o) { return o >= 0 && o < kNumRedOps; }

inline size_t dtype_size(DType d) {
  switch (d) {
    case DType::Int8: case DType::Uint8: return 1;
    case DType::Float16: case DType::Bfloat16: return 2;
    case DType::Int32: case DType::Uint32: case DType::Float32: return 4;
    case DType::Int64: case DType::Uint64: case DType::Float64: return 8;
  }
  return 0;
}

inline const char* dtype_name(DType d) {
  switch (d) {
    case DType::Int8: return "int8"; case DType::Uint8: return "uint8";
    case DType::Int32: return "int32"; case DType::Uint32: return "uint32";
    case DType::Int64: return "int64"; case DType::Uint64: return "uint64";
    case DType::Float16: return "fp16"; case DType::Float32: return "fp32";
    case DType::Float64: return "fp64"; case DType::Bfloat16: return "bf16";
  }
  return "?";
}

inline const char* op_name(RedOp o) {
  switch (o) {
    case RedOp::Sum: return "sum"; case RedOp::Prod: return "prod"; case RedOp::Max: return "max";
    case RedOp::Min: return "min"; case RedOp::Avg: return "avg";
  }
  return "?";
}

// ---- host-side bf16 / fp16 conversions, round-to-nearest-even, bit-identical
// to the device intrinsics (__float2bfloat16_rn / __float2half_rn).

inline float bf16_to_float(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

inline uint16_t float_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;  // NaN (canonical, as the device intrinsic)
  uint32_t lsb = (u >> 16) & 1u;
  u += 0x7fffu + lsb;
  return static_cast<uint16_t>(u >> 16);
}

inline float half_to_float(uint16_t h) {
  uint32_t sign = (h & 0x8000u) << 16;
  uint32_t exp = (h >> 10) & 0x1fu;
  uint32_t man = h & 0x3ffu;
  uint32_t u;
  if (exp == 0) {
    if (man == 0) {
      u = sign;
    } else {
      int e = -1;
      do { ++e; man <<= 1; } while ((man & 0x400u) == 0);
      man &= 0x3ffu;
      u = sign | ((127 - 15 - e) << 23) | (man << 13);
    }
  } else if (exp == 31) {
    u = sign | 0x7f800000u | (man << 13);
  } else {
    u = sign | ((exp + 127 - 15) << 23) | (man << 13);
  }
  float f;
  memcpy(&f, &u, 4);
  return f;
}

inline uint16_t float_to_half(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t absx = x & 0x7fffffffu;
  if (absx > 0x7f800000u) return 0x7fff;                              // NaN
  if (absx >= 0x477ff000u) return static_cast<uint16_t>(sign | 0x7c00u);  // overflow -> inf
  if (absx < 0x33000001u) return static_cast<uint16_t>(sign);         // underflow -> 0
  int32_t exp = static_cast<int32_t>(absx >> 23) - 127;
  uint32_t man = (absx & 0x7fffffu) | 0x800000u;
  uint32_t shift;
  uint32_t base;
  if (exp < -14) {  // subnormal half
    shift = static_cast<uint32_t>(13 + (-14 - exp));
    base = 0;
  } else {
    shift = 13;
    base = static_cast<uint32_t>(exp + 15 - 1) << 10;  // -1: the implicit bit adds one exponent step
  }
  uint32_t q = man >> shift;
  uint32_t rem = man & ((1u << shift) - 1u);
  uint32_t halfway = 1u << (shift - 1);
  if (rem > halfway || (rem == halfway && (q & 1u))) ++q;
  return static_cast<uint16_t>(sign | (base + q));
}

}  // namespace mnccl
