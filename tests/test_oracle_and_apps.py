"""The CPU oracle (against numpy / torch), the bf16 / fp16 conversions, the AVX2 verifier, and
the reference-shaped programs `app` and `perf_test` on the network data plane."""
import ctypes as C
import os
import subprocess
from pathlib import Path

import numpy as np
import pytest
import torch

from mini_nccl_b200 import _lib
from mini_nccl_b200.utils import oracle as O

ROOT = Path(__file__).resolve().parent.parent


def test_bf16_and_half_conversions_match_torch(lib):
    rng = np.random.default_rng(0)
    vals = np.concatenate([rng.standard_normal(4000).astype(np.float32) * s for s in (1e-8, 1e-4, 1.0, 300.0, 7e4)]
                          + [np.array([0.0, -0.0, 1.0, 65504.0, 65520.0, 1e-7, 6e-8, 2.9e-8, np.inf, -np.inf], np.float32)])
    t = torch.from_numpy(vals)
    want_bf = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    want_h = t.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    got_bf = np.array([lib.mnccl_float_to_bf16(float(v)) for v in vals], np.uint16)
    got_h = np.array([lib.mnccl_float_to_half(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got_bf, want_bf)
    assert np.array_equal(got_h, want_h)
    assert np.array_equal(O.f32_to_bf16_bits(vals), want_bf)
    back = np.array([lib.mnccl_half_to_float(int(h)) for h in want_h[:2000]], np.float32)
    assert np.array_equal(back, torch.from_numpy(want_h[:2000].view(np.int16)).view(torch.float16).float().numpy())


@pytest.mark.parametrize("dtype", list(range(10)))
@pytest.mark.parametrize("op", list(range(5)))
def test_oracle_against_wide_reference(dtype, op):
    n, count = 5, 2000
    ins = [O.make_input(dtype, count, r, op=op) for r in range(n)]
    got = O.oracle_allreduce(ins, dtype, op)
    ref = O.torch_fp32_reference(ins, dtype, op)
    if dtype in O.FLOAT_TYPES:
        tol = O.tolerance(dtype, n) * (8 if op == _lib.PROD else 1)
        assert np.abs(O.to_float64(got, dtype) - ref).max() <= tol
    else:
        bits = 8 * _lib.DTYPE_SIZES[dtype]
        want = [int(v) % (1 << bits) for v in ref]
        assert [int(v) % (1 << bits) for v in got] == want


def test_oracle_fp32_sum_is_rank_ordered():
    # (1e8 + 1) - 1e8 in fp32 depends on the order; rank order is the contract.
    a = [np.array([1e8], np.float32), np.array([1.0], np.float32), np.array([-1e8], np.float32)]
    assert O.oracle_allreduce(a, _lib.FLOAT32, _lib.SUM)[0] == np.float32(np.float32(np.float32(1e8) + np.float32(1)) - np.float32(1e8))


def test_avx2_verifier(lib):
    n = 1003
    a = np.random.default_rng(1).standard_normal(n).astype(np.float32)
    b = a.copy()
    bad = C.c_size_t()
    assert lib.mnccl_verify_f32(a.ctypes.data, b.ctypes.data, n, 1e-5, C.byref(bad)) == 0
    b[998] += 1e-3      # in the 8-wide body
    assert lib.mnccl_verify_f32(a.ctypes.data, b.ctypes.data, n, 1e-5, C.byref(bad)) == 1 and bad.value == 998
    b[998] = a[998]
    b[1002] = np.nan    # in the scalar tail, and a NaN must not pass
    assert lib.mnccl_verify_f32(a.ctypes.data, b.ctypes.data, n, 1e-5, C.byref(bad)) == 1 and bad.value == 1002
    ones = np.full(n, 3.0, np.float32)
    assert lib.mnccl_verify_const_f32(ones.ctypes.data, 3.0, n, 1e-5, C.byref(bad)) == 0
    ones[17] = 2.0
    assert lib.mnccl_verify_const_f32(ones.ctypes.data, 3.0, n, 1e-5, C.byref(bad)) == 1 and bad.value == 17
    s = np.empty(n, np.float32)
    lib.mnccl_sum_f32(a.ctypes.data, a.ctypes.data, s.ctypes.data, n)
    assert np.array_equal(s, a + a)


def _bin(name):
    exe = ROOT / "mini_nccl_b200" / "bin" / name
    if not exe.exists():
        from mini_nccl_b200 import build

        build.build()
    return str(exe)


@pytest.mark.skipif(torch.cuda.is_available(), reason="the no-GPU variant of the programs")
def test_app_and_perf_test_programs(free_port):
    env = dict(os.environ, MINI_NCCL_BOOTSTRAP_PORT=str(free_port), PERF_TEST_MAX_MIB="16")
    ps = [subprocess.Popen([_bin("app"), str(r), "127.0.0.1", "3"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
          for r in range(3)]
    outs = [p.communicate(timeout=120) for p in ps]
    assert all(p.returncode == 0 for p in ps), outs
    assert all("[PASS]" in o[0] and "= 6.0" in o[0] for o in outs)
    env["MINI_NCCL_BOOTSTRAP_PORT"] = str(free_port + 1)
    ps = [subprocess.Popen([_bin("perf_test"), str(r), "2", "127.0.0.1"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
          for r in range(2)]
    outs = [p.communicate(timeout=300) for p in ps]
    assert all(p.returncode == 0 for p in ps), outs
    table = outs[0][0]
    assert "Size(B)" in table and "AlgBW(GB/s)" in table and "BusBW(GB/s)" in table
    assert "1048576" in table and "16777216" in table and "(FAIL)" not in table
    assert subprocess.run([_bin("perf_test")], capture_output=True).returncode == 1  # usage


def test_dual_process_demo(free_port):
    env = dict(os.environ)
    ps = [subprocess.Popen([_bin("demo_dual_process"), role, "127.0.0.1", str(free_port)], env=env, stdout=subprocess.PIPE,
                           stderr=subprocess.PIPE, text=True) for role in ("server", "client")]
    outs = [p.communicate(timeout=60) for p in ps]
    assert all(p.returncode == 0 for p in ps), outs
    assert 'received: "Hello from the client' in outs[0][0] and 'received: "Hello from the server' in outs[1][0]
    assert subprocess.run([_bin("demo_dual_process")], capture_output=True).returncode == 1


def test_tensor_parallel_oracles_restates_the_kernels_arithmetic():
    """GEMM -> reduce-scatter and all-gather -> GEMM on the host: bf16 roundings where the kernels
    round, rank-ordered fp32 sum, rows partitioned by owner."""
    from mini_nccl_b200.utils import oracle as O

    rng = np.random.default_rng(7)
    n, M, N, K = 4, 64, 48, 96
    a = [O.f32_to_bf16_bits(rng.standard_normal((M, K // n)).astype(np.float32)) for _ in range(n)]
    b = [O.f32_to_bf16_bits(rng.standard_normal((N, K // n)).astype(np.float32)) for _ in range(n)]
    wide = sum(O.bf16_bits_to_f32(a[r]).astype(np.float64) @ O.bf16_bits_to_f32(b[r]).astype(np.float64).T for r in range(n))
    got = np.concatenate([O.bf16_bits_to_f32(O.oracle_gemm_reduce_scatter(a, b, r)) for r in range(n)])
    assert got.shape == (M, N)
    # n + 1 bf16 roundings of values of magnitude ~ sqrt(K): relative 2^-8 each
    assert np.abs(got - wide).max() <= (n + 1) * 2.0 ** -8 * np.abs(wide).max()
    # the partial products really are rounded before the sum: exact fp32 sums differ somewhere
    exact = O.bf16_bits_to_f32(O.f32_to_bf16_bits(wide.astype(np.float32)))
    assert np.any(got != exact)
    # one rank: reduce-scatter of one operand is the rounded product itself
    assert np.array_equal(O.oracle_gemm_reduce_scatter(a[:1], b[:1], 0), O.oracle_gemm_bf16(a[0], b[0]))
    # all-gather -> GEMM: gathered rows are the shards in rank order, product equals the plain GEMM
    x = [O.f32_to_bf16_bits(rng.standard_normal((M // n, K)).astype(np.float32)) for _ in range(n)]
    w = O.f32_to_bf16_bits(rng.standard_normal((N, K)).astype(np.float32))
    gathered, c = O.oracle_all_gather_gemm(x, w)
    assert gathered.shape == (M, K) and np.array_equal(gathered[M // n:2 * M // n], x[1])
    assert np.array_equal(c, O.oracle_gemm_bf16(np.concatenate(x), w))
    assert O.oracle_gemm_bf16(x[0], w, out_fp32=True).dtype == np.float32
