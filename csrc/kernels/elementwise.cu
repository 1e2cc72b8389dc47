// Elementwise pieces of the tensor-parallel block that sit between the two fused GEMM kernels.
//
// SwiGLU: the all-gather->GEMM kernel produces H[M, 2F] = (gate | up) for this rank's slice of the
// FFN; the GEMM->reduce-scatter kernel consumes act[M, F] = silu(gate) * up.  One pass: 16-byte
// loads of gate and up, fp32 math, one rounding to bf16, 16-byte store (3 bytes moved per output
// byte; a framework's silu followed by mul moves 5 and rounds twice).  The reference has no model
// code; this belongs to the tensor-parallel benchmark block (mini_nccl_b200/parallel/tp.py).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace {

__device__ __forceinline__ float silu(float x) { return x / (1.0f + __expf(-x)); }

__global__ void __launch_bounds__(256)
swiglu_bf16_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ act, int M, int F, long ldh, long lda) {
  const long vec_per_row = F / 8;
  const long total = static_cast<long>(M) * vec_per_row;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long m = i / vec_per_row;
    const long v = i - m * vec_per_row;
    const __nv_bfloat16* row = h + m * ldh;
    const uint4 g = *reinterpret_cast<const uint4*>(row + v * 8);
    const uint4 u = *reinterpret_cast<const uint4*>(row + F + v * 8);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g);
    const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u);
    uint4 y;
    __nv_bfloat162* yp = reinterpret_cast<__nv_bfloat162*>(&y);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 gf = __bfloat1622float2(gp[k]);
      const float2 uf = __bfloat1622float2(up[k]);
      yp[k] = __floats2bfloat162_rn(silu(gf.x) * uf.x, silu(gf.y) * uf.y);
    }
    *reinterpret_cast<uint4*>(act + m * lda + v * 8) = y;
  }
}

}  // namespace

extern "C" {
#define MNCCL_EXPORT __attribute__((visibility("default")))

// act[M, F] = silu(h[:, 0:F]) * h[:, F:2F]; bf16 in and out, row strides ldh / lda in elements
// (0 = dense: 2F and F).  F, ldh and lda must be multiples of 8 and both pointers 16-byte aligned.
// Returns 0, a negative code for bad arguments, or a cudaError_t + 1000.
MNCCL_EXPORT int mncclSwiGluBf16(const void* h, void* act, int M, int F, long ldh, long lda, cudaStream_t stream) {
  if (h == nullptr || act == nullptr || M <= 0 || F <= 0) return -1;
  if (ldh == 0) ldh = 2L * F;
  if (lda == 0) lda = F;
  if (F % 8 != 0 || ldh % 8 != 0 || lda % 8 != 0 || ldh < 2L * F || lda < F) return -2;
  if ((reinterpret_cast<uintptr_t>(h) & 15u) != 0 || (reinterpret_cast<uintptr_t>(act) & 15u) != 0) return -2;
  const long total = static_cast<long>(M) * (F / 8);
  long blocks = (total + 255) / 256;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) sms = 148;
  if (blocks > 8L * sms) blocks = 8L * sms;
  swiglu_bf16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h),
                                                                        static_cast<__nv_bfloat16*>(act), M, F, ldh, lda);
  const cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : static_cast<int>(e) + 1000;
}

}  // extern "C"
