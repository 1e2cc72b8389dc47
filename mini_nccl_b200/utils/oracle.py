"""Host-side data generation and oracles shared by the tests, the benchmarks
and the examples.  Inputs are seeded per rank (seed + rank), as the benchmark
configurations require; the oracle is the library's C++ restatement of the
device arithmetic (rank-ordered, fp32 accumulation, one final rounding), so
P2P results can be compared bit for bit.  The reference checks its results
against a constant only (reference: tests/perf_test.cpp:102-134), which hides
ordering and staleness bugs; seeded random data does not.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from .. import _lib

NP_DTYPES = {
    _lib.INT8: np.int8, _lib.UINT8: np.uint8, _lib.INT32: np.int32, _lib.UINT32: np.uint32,
    _lib.INT64: np.int64, _lib.UINT64: np.uint64, _lib.FLOAT16: np.float16, _lib.FLOAT32: np.float32,
    _lib.FLOAT64: np.float64, _lib.BFLOAT16: np.uint16,  # bf16 travels as raw bits on the host
}
DTYPE_NAMES = {
    _lib.INT8: "int8", _lib.UINT8: "uint8", _lib.INT32: "int32", _lib.UINT32: "uint32", _lib.INT64: "int64",
    _lib.UINT64: "uint64", _lib.FLOAT16: "fp16", _lib.FLOAT32: "fp32", _lib.FLOAT64: "fp64", _lib.BFLOAT16: "bf16",
}
OP_NAMES = {_lib.SUM: "sum", _lib.PROD: "prod", _lib.MAX: "max", _lib.MIN: "min", _lib.AVG: "avg"}
FLOAT_TYPES = (_lib.FLOAT16, _lib.FLOAT32, _lib.FLOAT64, _lib.BFLOAT16)


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    lsb = (u >> 16) & 1
    return ((u + 0x7FFF + lsb) >> 16).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << 16).view(np.float32)


def make_input(dtype: int, count: int, rank: int, seed: int = 1234, op: int = _lib.SUM, dist: str = "uniform") -> np.ndarray:
    """Per-rank seeded input as a host array in the dtype's storage type."""
    rng = np.random.default_rng(seed + rank)
    if dtype in FLOAT_TYPES:
        if op == _lib.PROD:
            x = rng.uniform(0.5, 1.5, count)
        elif dist == "normal":
            x = rng.standard_normal(count)
        else:
            x = rng.uniform(-1.0, 1.0, count)
        if dtype == _lib.BFLOAT16:
            return f32_to_bf16_bits(x.astype(np.float32))
        return x.astype(NP_DTYPES[dtype])
    np_t = NP_DTYPES[dtype]
    if op == _lib.PROD:
        lo, hi = (1, 3)
    elif np.issubdtype(np_t, np.signedinteger):
        lo, hi = (-6, 7) if np_t == np.int8 else (-1000, 1000)
    else:
        lo, hi = (0, 13) if np_t == np.uint8 else (0, 2000)
    return rng.integers(lo, hi, count, dtype=np.int64).astype(np_t)


def oracle_allreduce(inputs: list[np.ndarray], in_dtype: int, op: int, wire_dtype: int | None = None,
                     out_dtype: int | None = None, scale: float = 1.0) -> np.ndarray:
    """Rank-ordered host reduction through the library's C++ oracle."""
    wire_dtype = in_dtype if wire_dtype is None else wire_dtype
    out_dtype = in_dtype if out_dtype is None else out_dtype
    n = len(inputs)
    count = inputs[0].size
    keep = [np.ascontiguousarray(a) for a in inputs]
    ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in keep])
    out = np.empty(count, dtype=NP_DTYPES[out_dtype])
    rc = _lib.lib().mnccl_oracle_allreduce(in_dtype, wire_dtype, out_dtype, op, n, ptrs, out.ctypes.data, count, float(scale))
    if rc != 0:
        raise RuntimeError(f"oracle failed with {rc}")
    return out


def to_float64(a: np.ndarray, dtype: int) -> np.ndarray:
    if dtype == _lib.BFLOAT16:
        return bf16_bits_to_f32(a).astype(np.float64)
    return a.astype(np.float64)


def torch_fp32_reference(inputs: list[np.ndarray], dtype: int, op: int, scale: float = 1.0):
    """Plain PyTorch fp32 (fp64 for fp64 / 64-bit integers) reference of the same reduction."""
    import torch

    wide = torch.float64 if dtype in (_lib.FLOAT64, _lib.INT64, _lib.UINT64, _lib.INT32, _lib.UINT32) else torch.float32
    stack = torch.stack([torch.from_numpy(to_float64(a, dtype)).to(wide) for a in inputs])
    if op in (_lib.SUM, _lib.AVG):
        r = stack.sum(0)
        if op == _lib.AVG:
            r = r / len(inputs)
            if dtype not in FLOAT_TYPES:
                r = torch.trunc(r)
    elif op == _lib.PROD:
        r = stack.prod(0)
    elif op == _lib.MAX:
        r = stack.max(0).values
    else:
        r = stack.min(0).values
    return (r * scale).to(torch.float64).numpy()


def tolerance(dtype: int, nranks: int) -> float:
    """Absolute tolerance against the wide reference for inputs of magnitude <= ~1.5."""
    if dtype == _lib.BFLOAT16:
        return 0.04 * max(1, nranks // 2)
    if dtype == _lib.FLOAT16:
        return 0.006 * max(1, nranks // 2)
    if dtype == _lib.FLOAT32:
        return 1e-5 * nranks
    if dtype == _lib.FLOAT64:
        return 1e-12 * nranks
    return 0.0


# --------------------------------------------------------------------------- tensor-parallel fusions
# Host restatements of the three GEMM kernels, in the kernels' own arithmetic: bf16 operands (as
# uint16 bit patterns), products and sums in fp32, ONE rounding to bf16 where the kernel rounds.
# The tensor cores add the K products of a tile in an order of their own, so GPU results are
# compared with a tolerance; the roundings and the rank order of the reduction are exact.

def oracle_gemm_bf16(a_bits: np.ndarray, b_bits: np.ndarray, out_fp32: bool = False) -> np.ndarray:
    """``C[M, N] = A[M, K] @ B[N, K].T``: bf16 bit patterns in, fp32 accumulation, bf16 bit patterns
    (or fp32 values) out."""
    acc = bf16_bits_to_f32(np.ascontiguousarray(a_bits)) @ bf16_bits_to_f32(np.ascontiguousarray(b_bits)).T
    acc = acc.astype(np.float32)
    return acc if out_fp32 else f32_to_bf16_bits(acc)


def oracle_gemm_reduce_scatter(a_bits: list[np.ndarray], b_bits: list[np.ndarray], rank: int, return_sum: bool = False):
    """GEMM -> reduce-scatter as the fused kernel computes it: every rank's partial product is rounded
    to bf16 before it travels, the owner adds the partial tiles in RANK ORDER in fp32 and rounds the sum
    once.  ``a_bits[r]`` is ``[M, K_r]``, ``b_bits[r]`` is ``[N, K_r]``; returns the rows ``rank`` owns
    (with ``return_sum`` also the fp32 sum before its rounding)."""
    n = len(a_bits)
    M = a_bits[0].shape[0]
    if M % n:
        raise ValueError("M must divide by the number of ranks")
    per = M // n
    rows = slice(rank * per, (rank + 1) * per)
    acc = None
    for r in range(n):
        partial = bf16_bits_to_f32(oracle_gemm_bf16(a_bits[r][rows], b_bits[r]))  # what rank r sends
        acc = partial.copy() if acc is None else (acc + partial).astype(np.float32)
    return (f32_to_bf16_bits(acc), acc) if return_sum else f32_to_bf16_bits(acc)


def oracle_all_gather_gemm(x_shards_bits: list[np.ndarray], b_bits: np.ndarray) -> tuple[np.ndarray, np.ndarray]:
    """all-gather -> GEMM: the gathered activations (row-wise concatenation of the shards, which must be
    bit-identical on every rank) and their product with this rank's weight slice ``b [N_r, K]``."""
    gathered = np.concatenate([np.ascontiguousarray(s) for s in x_shards_bits], axis=0)
    return gathered, oracle_gemm_bf16(gathered, b_bits)
