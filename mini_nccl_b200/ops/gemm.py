"""bf16 GEMM on the Blackwell tensor cores (tcgen05.mma, accumulators in tensor memory, operands
staged by TMA): ``C = A @ B.T`` with ``A [M, K]`` and ``B [N, K]`` row-major, the layout of an
``nn.Linear`` weight.  Fails loudly when the native kernel is missing: there is no fallback."""
from __future__ import annotations

import ctypes as C

from .._lib import lib


def _native():
    L = lib()
    if not hasattr(L, "mncclGemmBf16"):
        raise RuntimeError("libmini_nccl.so was built without the sm_100a GEMM (csrc/kernels/gemm_sm100.cu)")
    return L


def gemm_bf16(a, b, out=None, out_dtype=None, stream=None):
    """``out[M, N] = a[M, K] @ b[N, K].T``; ``a`` and ``b`` bf16 with a unit inner stride."""
    import torch

    if a.dtype != torch.bfloat16 or b.dtype != torch.bfloat16:
        raise TypeError("gemm_bf16 needs bf16 operands")
    if a.dim() != 2 or b.dim() != 2 or a.shape[1] != b.shape[1]:
        raise ValueError("shapes: a [M, K], b [N, K]")
    if a.stride(1) != 1 or b.stride(1) != 1:
        raise ValueError("operands need a unit inner stride")
    M, K = a.shape
    N = b.shape[0]
    out_dtype = out_dtype or (out.dtype if out is not None else torch.bfloat16)
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype, device=a.device)
    if out.dtype not in (torch.bfloat16, torch.float32) or out.stride(1) != 1 or tuple(out.shape) != (M, N):
        raise ValueError("out must be [M, N] bf16 or fp32 with a unit inner stride")
    s = stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream
    rc = _native().mncclGemmBf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), M, N, K, a.stride(0), b.stride(0), out.stride(0),
                                 1 if out.dtype == torch.float32 else 0, s)
    if rc != 0:
        raise RuntimeError(f"mncclGemmBf16 failed with code {rc}")
    return out


def gemm_status() -> int:
    """Error word of the GEMM kernels on the current device (0 = every bounded wait completed); clears it."""
    st = C.c_uint32()
    rc = _native().mncclGemmStatus(C.byref(st))
    if rc != 0:
        raise RuntimeError(f"mncclGemmStatus failed with code {rc}")
    return st.value


def set_pair_mode(mode: int) -> None:
    """-1: automatic; 0: single-CTA 128 x 256 tiles; 1: CTA pairs (tcgen05 cta_group::2, 256 x 256 tiles)."""
    _native().mncclGemmSetPairMode(int(mode))


def gemm_plan(M: int, N: int, ctas: int = 148, narrow: bool = True):
    """``(tile_n, pair)``: the tile width the single-CTA kernel would use for an ``M x N`` product on
    ``ctas`` CTAs and whether the CTA-pair kernel would be taken instead.  Host logic only; needs no GPU."""
    import ctypes as C

    tile_n, pair = C.c_int(0), C.c_int(0)
    _native().mncclGemmPlan(int(M), int(N), int(ctas), 1 if narrow else 0, C.byref(tile_n), C.byref(pair))
    return tile_n.value, bool(pair.value)
