"""Elementwise kernels of the tensor-parallel block (csrc/kernels/elementwise.cu)."""
from __future__ import annotations

from .._lib import lib


def swiglu_bf16(h, out=None, stream=None):
    """``out[M, F] = silu(h[:, :F]) * h[:, F:]`` for a bf16 ``h [M, 2F]`` (gate | up): one pass, fp32
    math, one rounding.  ``h`` and ``out`` need a unit inner stride, 16-byte aligned rows and F % 8 == 0."""
    import torch

    L = lib()
    if not hasattr(L, "mncclSwiGluBf16"):
        raise RuntimeError("libmini_nccl.so was built without csrc/kernels/elementwise.cu")
    if h.dtype != torch.bfloat16 or h.dim() != 2 or h.shape[1] % 2 or h.stride(1) != 1:
        raise TypeError("h must be a bf16 matrix [M, 2F] with a unit inner stride")
    M, F = h.shape[0], h.shape[1] // 2
    if out is None:
        out = torch.empty((M, F), dtype=torch.bfloat16, device=h.device)
    if out.dtype != torch.bfloat16 or tuple(out.shape) != (M, F) or out.stride(1) != 1:
        raise TypeError("out must be a bf16 matrix [M, F] with a unit inner stride")
    s = stream.cuda_stream if stream is not None else torch.cuda.current_stream().cuda_stream
    rc = L.mncclSwiGluBf16(h.data_ptr(), out.data_ptr(), M, F, h.stride(0), out.stride(0), s)
    if rc != 0:
        raise RuntimeError(f"mncclSwiGluBf16 failed with code {rc}")
    return out
