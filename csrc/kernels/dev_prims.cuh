// Device primitives for the sm_100a collective kernels: system-scope flag
// loads / stores, the bounded wait, the cross-rank per-block barrier, typed
// 16-byte vector I/O with fp32 accumulation, and the multimem (NVLS) wrappers.
//
// Counterparts in the reference: wait_kernel / set_flag_kernel, one launch per
// slice, polling host-pinned flags (reference: src/mini_nccl.cu:22-36), and the
// scalar elementwise_reduce_kernel (reference: src/mini_nccl.cu:43-47).  Here
// waits and signals are inline in the data kernels, flags are in device memory
// and every wait is bounded: it gives up after spin_timeout_ns or when the
// abort word is set, records a status and lets the kernel return.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "kernels/comm_dev.h"

namespace mnccl {
namespace dev {

// ------------------------------------------------------------ memory ops

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_volatile_u32(const volatile uint32_t* p) {
  uint32_t v;
  asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_u32(volatile uint32_t* p, uint32_t v) {
  asm volatile("st.volatile.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
// 16-byte load that is cached in L2 only: for buffers whose lines this SM may hold from an earlier use.
__device__ __forceinline__ uint4 ld_cg_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_volatile_v4(void* p, uint4 v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// ------------------------------------------------------------ control block

struct BlockCtl {        // one per thread block, in shared memory
  uint32_t epoch;        // this block's barrier epoch (cached from LocalState)
  uint32_t ll_seq;
  volatile uint32_t fail;  // DevStatus of the first failed wait in this block
  // pipelined kernel (pipe_body): worker warps that have finished the block's i-th chunk (ring of 4),
  // chunks of this block whose inputs the poller has seen, chunks the publisher has published
  volatile uint32_t pipe_done[4];
  volatile uint32_t pipe_ready;
  volatile uint32_t pipe_pub;
};

__device__ __forceinline__ LocalState* local_state(const CommDev& c) {
  return reinterpret_cast<LocalState*>(c.ctrl[c.rank] + c.off_local);
}
__device__ __forceinline__ uint32_t* sig_slot(const CommDev& c, int owner, int blk, int src) {
  return reinterpret_cast<uint32_t*>(c.ctrl[owner] + c.off_sig) + (blk * kMaxRanks + src);
}

__device__ __forceinline__ void record_failure(const CommDev& c, uint32_t code, uint32_t detail) {
  LocalState* ls = local_state(c);
  if (atomicCAS(&ls->status, 0u, code) == 0u) {
    ls->detail = detail;
    if (c.host_progress) {
      st_volatile_u32(c.host_progress + 3, detail);
      __threadfence_system();
      st_volatile_u32(c.host_progress + 2, code);
    }
  }
}

// Checked build (-DMNCCL_DEVICE_CHECKS=1, libmini_nccl_devcheck.so): every access to a staging area
// is tested against the area's size and the 16-byte alignment first; a bad one is RECORDED in the
// status word (kDevBadIndex, detail = offset / 16) and skipped -- never a trap, never the access.
// The product build compiles the test away.  (compute-sanitizer is not available everywhere this
// library is developed; these checks and the host oracle stand in for it.)
#ifdef MNCCL_DEVICE_CHECKS
__device__ __forceinline__ bool stage_access_ok(const CommDev& c, uint64_t off, uint32_t bytes) {
  if (off + bytes <= c.stage_bytes && (off & 15u) == 0u) return true;
  record_failure(c, kDevBadIndex, static_cast<uint32_t>(off >> 4));
  return false;
}
#define MNCCL_STAGE_OK(c, off, bytes) ::mnccl::dev::stage_access_ok((c), (off), (bytes))
#else
#define MNCCL_STAGE_OK(c, off, bytes) true
#endif

// Waits until *p >= target (wrap-safe).  Returns kDevOk, kDevTimeout or
// kDevAborted; never spins for longer than c.spin_timeout_ns.
__device__ __forceinline__ uint32_t wait_ge(const uint32_t* p, uint32_t target, const CommDev& c) {
  if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return kDevOk;
  const uint64_t t0 = globaltimer_ns();
  for (uint32_t it = 1;; ++it) {
    if (static_cast<int32_t>(ld_acquire_sys(p) - target) >= 0) return kDevOk;
    if ((it & 255u) == 0u) {
      if (c.abort_word != nullptr && ld_volatile_u32(c.abort_word) != 0u) return kDevAborted;
      if (globaltimer_ns() - t0 > c.spin_timeout_ns) return kDevTimeout;
    }
  }
}

// Kernel prologue: every thread calls it once, first thing.
__device__ __forceinline__ void block_begin(const CommDev& c, int blk, BlockCtl& ctl) {
  if (threadIdx.x == 0) {
    LocalState* ls = local_state(c);
    ctl.epoch = ls->epoch[blk];
    // ONE LL sequence per communicator (word 0), read by every block: inbox slots are addressed by unit
    // offset, not by block, so a per-block sequence would go wrong as soon as two LL calls split their
    // units over a different number of blocks (a block could meet a stale packet carrying the very
    // flag it waits for).
    ctl.ll_seq = ls->ll_seq[0];
    ctl.fail = 0;
    for (int i = 0; i < 4; ++i) ctl.pipe_done[i] = 0;
    ctl.pipe_ready = 0;
    ctl.pipe_pub = 0;
    if (blk == 0) {
      uint32_t s = ls->started + 1;
      ls->started = s;
      if (c.host_progress) st_volatile_u32(c.host_progress + 0, s);
    }
  }
  __syncthreads();
}

// Kernel epilogue: every thread calls it once, last thing.
__device__ __forceinline__ void block_end(const CommDev& c, int blk, int nblk, BlockCtl& ctl) {
  __syncthreads();
  if (threadIdx.x == 0) {
    LocalState* ls = local_state(c);
    ls->epoch[blk] = ctl.epoch;
    __threadfence();
    uint32_t t = atomicAdd(&ls->ticket, 1u);
    if (t == static_cast<uint32_t>(nblk - 1)) {
      ls->ticket = 0;
      ls->ll_seq[0] = ctl.ll_seq;  // every block of an LL kernel holds the same new value; others leave it unchanged
      uint32_t d = ls->done + 1;
      ls->done = d;
      if (c.host_progress) st_volatile_u32(c.host_progress + 1, d);
    }
  }
}

// Cross-rank barrier between the blocks with index `blk` of every rank.  All
// threads of the block must call it.  Writes made by any thread of this block
// before the call (local or to peer memory) are visible to the peers' block
// `blk` after their call returns.  Returns false after a failed wait; the
// caller must then skip to block_end.
__device__ __forceinline__ bool block_barrier(const CommDev& c, int blk, BlockCtl& ctl) {
  __syncthreads();
  const uint32_t e = ctl.epoch + 1;
  const int t = threadIdx.x;
  if (t < c.nranks && t != c.rank) {
    st_release_sys(sig_slot(c, t, blk, c.rank), e);
    uint32_t r = wait_ge(sig_slot(c, c.rank, blk, t), e, c);
    if (r != kDevOk) {
      ctl.fail = r;
      record_failure(c, r, (static_cast<uint32_t>(blk) << 16) | static_cast<uint32_t>(t));
    }
  }
  __syncthreads();
  if (t == 0) ctl.epoch = e;  // read again only after the next __syncthreads
  return ctl.fail == 0;
}

// ------------------------------------------------------------ element types

template <typename T> struct Elem;  // Raw storage, accumulator, conversions

#define MNCCL_INT_ELEM(T)                                                   \
  template <> struct Elem<T> {                                              \
    using Raw = T;                                                          \
    using Acc = T;                                                          \
    static constexpr bool kFloat = false;                                   \
    __device__ __forceinline__ static Acc up(Raw r) { return r; }           \
    __device__ __forceinline__ static Raw down(Acc a) { return a; }         \
  };
MNCCL_INT_ELEM(int8_t)
MNCCL_INT_ELEM(uint8_t)
MNCCL_INT_ELEM(uint16_t)
MNCCL_INT_ELEM(int32_t)
MNCCL_INT_ELEM(uint32_t)
MNCCL_INT_ELEM(int64_t)
MNCCL_INT_ELEM(uint64_t)
#undef MNCCL_INT_ELEM

template <> struct Elem<float> {
  using Raw = float;
  using Acc = float;
  static constexpr bool kFloat = true;
  __device__ __forceinline__ static Acc up(Raw r) { return r; }
  __device__ __forceinline__ static Raw down(Acc a) { return a; }
};
template <> struct Elem<double> {
  using Raw = double;
  using Acc = double;
  static constexpr bool kFloat = true;
  __device__ __forceinline__ static Acc up(Raw r) { return r; }
  __device__ __forceinline__ static Raw down(Acc a) { return a; }
};
template <> struct Elem<__half> {
  using Raw = uint16_t;
  using Acc = float;
  static constexpr bool kFloat = true;
  __device__ __forceinline__ static Acc up(Raw r) { return __half2float(__ushort_as_half(r)); }
  __device__ __forceinline__ static Raw down(Acc a) { return __half_as_ushort(__float2half_rn(a)); }
};
template <> struct Elem<__nv_bfloat16> {
  using Raw = uint16_t;
  using Acc = float;
  static constexpr bool kFloat = true;
  __device__ __forceinline__ static Acc up(Raw r) { return __bfloat162float(__ushort_as_bfloat16(r)); }
  __device__ __forceinline__ static Raw down(Acc a) { return __bfloat16_as_ushort(__float2bfloat16_rn(a)); }
};

// Reduction operators on accumulators.  0 Sum, 1 Prod, 2 Max, 3 Min (Avg is
// Sum plus a final factor).
template <int OP, typename A>
__device__ __forceinline__ A combine(A a, A b) {
  if (OP == 0) return a + b;
  if (OP == 1) return a * b;
  if (OP == 2) return a > b ? a : b;
  return a < b ? a : b;
}

template <typename OutT, typename A>
__device__ __forceinline__ A finalize(A acc, const CollArgs& a) {
  if constexpr (sizeof(A) == 8 && Elem<OutT>::kFloat) {
    return a.scale_d != 1.0 ? acc * a.scale_d : acc;
  } else if constexpr (Elem<OutT>::kFloat) {
    return a.scale_f != 1.0f ? acc * a.scale_f : acc;
  } else {
    return a.int_div > 1 ? static_cast<A>(acc / static_cast<A>(a.int_div)) : acc;
  }
}

// ------------------------------------------------------------ vector I/O
// A "vector" is VW consecutive elements; VW * sizeof(wire type) == 16 bytes.

template <int BYTES> struct RawVec {
  uint4 q[BYTES / 16];
};
template <> struct RawVec<8> {
  uint2 q[1];
};
template <> struct RawVec<4> {
  uint32_t q[1];
};

template <typename T, int VW>
__device__ __forceinline__ void load_vec(const void* base, uint64_t i0, uint64_t limit, bool aligned,
                                         typename Elem<T>::Acc (&v)[VW]) {
  using Raw = typename Elem<T>::Raw;
  constexpr int NB = VW * sizeof(Raw);
  const Raw* p = static_cast<const Raw*>(base);
  if (aligned && i0 + VW <= limit) {
    union {
      RawVec<NB> vec;
      Raw e[VW];
    } u;
    if constexpr (NB >= 16) {
      const uint4* src = reinterpret_cast<const uint4*>(p + i0);
#pragma unroll
      for (int j = 0; j < NB / 16; ++j) u.vec.q[j] = src[j];
    } else {
      u.vec.q[0] = *reinterpret_cast<const uint2*>(p + i0);
    }
#pragma unroll
    for (int k = 0; k < VW; ++k) v[k] = Elem<T>::up(u.e[k]);
  } else {
#pragma unroll
    for (int k = 0; k < VW; ++k) v[k] = (i0 + k < limit) ? Elem<T>::up(p[i0 + k]) : typename Elem<T>::Acc(0);
  }
}

template <typename T, int VW>
__device__ __forceinline__ void store_vec(void* base, uint64_t i0, uint64_t limit, bool aligned,
                                          const typename Elem<T>::Acc (&v)[VW]) {
  using Raw = typename Elem<T>::Raw;
  constexpr int NB = VW * sizeof(Raw);
  Raw* p = static_cast<Raw*>(base);
  if (aligned && i0 + VW <= limit) {
    union {
      RawVec<NB> vec;
      Raw e[VW];
    } u;
#pragma unroll
    for (int k = 0; k < VW; ++k) u.e[k] = Elem<T>::down(v[k]);
    if constexpr (NB >= 16) {
      uint4* dst = reinterpret_cast<uint4*>(p + i0);
#pragma unroll
      for (int j = 0; j < NB / 16; ++j) dst[j] = u.vec.q[j];
    } else {
      *reinterpret_cast<uint2*>(p + i0) = u.vec.q[0];
    }
  } else {
#pragma unroll
    for (int k = 0; k < VW; ++k)
      if (i0 + k < limit) p[i0 + k] = Elem<T>::down(v[k]);
  }
}

// Pack VW accumulators into VW raw elements (NB bytes) and back.
template <typename T, int VW>
struct Packed {
  using Raw = typename Elem<T>::Raw;
  static constexpr int NB = VW * sizeof(Raw);
  union {
    RawVec<NB> vec;
    Raw e[VW];
    uint32_t w[NB / 4];
  };
  __device__ __forceinline__ void from_acc(const typename Elem<T>::Acc (&v)[VW]) {
#pragma unroll
    for (int k = 0; k < VW; ++k) e[k] = Elem<T>::down(v[k]);
  }
  __device__ __forceinline__ void to_acc(typename Elem<T>::Acc (&v)[VW]) const {
#pragma unroll
    for (int k = 0; k < VW; ++k) v[k] = Elem<T>::up(e[k]);
  }
};

// ------------------------------------------------------------ multimem (NVLS)

template <typename T> struct Nvls {
  static constexpr bool kSupported = false;
};
template <> struct Nvls<float> {
  static constexpr bool kSupported = true;
  __device__ __forceinline__ static uint4 ld_reduce_add(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
};
template <> struct Nvls<__nv_bfloat16> {
  static constexpr bool kSupported = true;
  __device__ __forceinline__ static uint4 ld_reduce_add(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
};
template <> struct Nvls<__half> {
  static constexpr bool kSupported = true;
  __device__ __forceinline__ static uint4 ld_reduce_add(const void* mc) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
  }
};

// 16-byte multicast store: the switch writes the same 16 bytes to every rank.
__device__ __forceinline__ void multimem_st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ bool is_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// True when vectors of VW elements of T starting at `p` can use wide accesses:
// 8-byte alignment for 8-byte vectors, 16-byte alignment otherwise.
template <typename T, int VW>
__device__ __forceinline__ bool vec_aligned(const void* p) {
  constexpr unsigned NB = VW * sizeof(typename Elem<T>::Raw);
  constexpr unsigned mask = (NB >= 16 ? 16u : NB) - 1u;
  return (reinterpret_cast<uintptr_t>(p) & mask) == 0;
}

}  // namespace dev
}  // namespace mnccl
