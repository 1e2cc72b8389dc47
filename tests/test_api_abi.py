"""The C ABI contract: enum values, error strings, argument checks, the exception firewall.
Mirrors what callers of the reference can rely on (reference: include/mini_nccl_api.h:15-69,
src/api.cpp:14-26,28-66,136-190)."""
import ctypes as C
import re
from pathlib import Path

import numpy as np
import pytest

from mini_nccl_b200 import _lib

ROOT = Path(__file__).resolve().parent.parent


def test_error_strings(lib):
    want = ["no error", "unhandled cuda error", "system error", "internal error", "invalid argument", "invalid usage",
            "remote error", "in progress"]
    for code, text in enumerate(want):
        assert lib.ncclGetErrorString(code).decode() == text
        assert lib.mncclGetErrorString(code).decode() == text
    assert lib.ncclGetErrorString(99).decode() == "unknown error"


def test_header_enum_values():
    h = (ROOT / "include" / "mini_nccl_api.h").read_text()
    for name, val in [("ncclSuccess", 0), ("ncclUnhandledCudaError", 1), ("ncclSystemError", 2), ("ncclInternalError", 3),
                      ("ncclInvalidArgument", 4), ("ncclInvalidUsage", 5), ("ncclRemoteError", 6), ("ncclInProgress", 7),
                      ("ncclInt8", 0), ("ncclUint8", 1), ("ncclInt32", 2), ("ncclUint32", 3), ("ncclInt64", 4),
                      ("ncclUint64", 5), ("ncclFloat16", 6), ("ncclFloat", 7), ("ncclDouble", 8), ("ncclBfloat16", 9),
                      ("ncclSum", 0), ("ncclProd", 1), ("ncclMax", 2), ("ncclMin", 3), ("ncclAvg", 4)]:
        assert re.search(rf"\b{name}\s*=\s*{val}\b", h), name
    for fn in ("ncclGetErrorString", "ncclCommInitRank", "ncclCommDestroy", "ncclCommUserRank", "ncclCommCount", "ncclAllReduce"):
        assert re.search(rf"\b{fn}\s*\(", h), fn
    assert "const char* ip" in h  # init takes the root / master address, not a ncclUniqueId


def test_null_and_range_arguments(lib):
    comm = C.c_void_p()
    assert lib.ncclCommInitRank(None, 2, 0, b"127.0.0.1") == _lib.INVALID_ARGUMENT
    assert lib.ncclCommInitRank(C.byref(comm), 2, 2, b"127.0.0.1") == _lib.INVALID_ARGUMENT
    assert lib.ncclCommInitRank(C.byref(comm), 2, -2, b"127.0.0.1") == _lib.INVALID_ARGUMENT
    assert lib.ncclCommInitRank(C.byref(comm), 0, 0, b"127.0.0.1") == _lib.INVALID_ARGUMENT
    assert lib.ncclCommDestroy(None) == _lib.INVALID_ARGUMENT
    r = C.c_int()
    assert lib.ncclCommUserRank(None, C.byref(r)) == _lib.INVALID_ARGUMENT
    assert lib.ncclCommCount(None, C.byref(r)) == _lib.INVALID_ARGUMENT
    x = np.zeros(4, np.float32)
    assert lib.ncclAllReduce(x.ctypes.data, x.ctypes.data, 4, _lib.FLOAT32, _lib.SUM, None, None) == _lib.INVALID_ARGUMENT


def test_single_rank_communicator_on_host(lib, free_port, monkeypatch):
    # One rank, no GPU: init (NULL ip means 127.0.0.1), queries, AllReduce of one operand, destroy.
    import os

    os.environ["MINI_NCCL_BOOTSTRAP_PORT"] = str(free_port)
    comm = C.c_void_p()
    assert lib.ncclCommInitRank(C.byref(comm), 1, 0, None) == 0
    r, n = C.c_int(-1), C.c_int(-1)
    assert lib.ncclCommUserRank(comm, C.byref(r)) == 0 and r.value == 0
    assert lib.ncclCommCount(comm, C.byref(n)) == 0 and n.value == 1
    assert lib.ncclCommUserRank(comm, None) == _lib.INVALID_ARGUMENT
    x = np.arange(10, dtype=np.float32)
    y = np.zeros_like(x)
    assert lib.ncclAllReduce(None, y.ctypes.data, 10, _lib.FLOAT32, _lib.SUM, comm, None) == _lib.INVALID_ARGUMENT
    assert lib.ncclAllReduce(x.ctypes.data, None, 10, _lib.FLOAT32, _lib.SUM, comm, None) == _lib.INVALID_ARGUMENT
    assert lib.ncclAllReduce(x.ctypes.data, y.ctypes.data, 0, _lib.FLOAT32, _lib.SUM, comm, None) == 0  # count 0: success
    assert lib.ncclAllReduce(x.ctypes.data, y.ctypes.data, 10, 17, _lib.SUM, comm, None) == _lib.INVALID_ARGUMENT
    assert lib.ncclAllReduce(x.ctypes.data, y.ctypes.data, 10, _lib.FLOAT32, 9, comm, None) == _lib.INVALID_ARGUMENT
    import torch

    if not torch.cuda.is_available():
        for dtype in range(10):  # every declared type works, including those the reference rejects
            for op in range(5):
                a = np.frombuffer(np.random.default_rng(dtype).bytes(64 * _lib.DTYPE_SIZES[dtype]), dtype=np.uint8).copy()
                if dtype in (_lib.FLOAT16, _lib.FLOAT32, _lib.FLOAT64, _lib.BFLOAT16):
                    a[:] = 0x3C  # finite values only
                b = np.zeros_like(a)
                assert lib.ncclAllReduce(a.ctypes.data, b.ctypes.data, 64, dtype, op, comm, None) == 0
                assert np.array_equal(a, b)
        st = C.create_string_buffer(4096)
        assert lib.mncclCommStats(comm, st, 4096) == 0
        assert b'"plane":"soft"' in st.value
    err = C.c_int(-1)
    assert lib.mncclCommGetAsyncError(comm, C.byref(err)) == 0 and err.value == 0
    assert lib.ncclCommDestroy(comm) == 0


def test_init_failure_is_an_error_code_not_an_exception(lib, free_port):
    # Nobody listens at the root address: the exception stays behind the firewall.
    import os

    os.environ["MINI_NCCL_BOOTSTRAP_PORT"] = str(free_port)
    os.environ["MINI_NCCL_CONNECT_RETRIES"] = "1"
    from mini_nccl_b200 import _lib as L

    # A fresh process reads the environment at its first use of the config.
    import subprocess
    import sys

    code = ("import ctypes as C, mini_nccl_b200 as m; c=C.c_void_p(); "
            "print('RC', m.lib().ncclCommInitRank(C.byref(c), 2, 1, b'127.0.0.1'))")
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, cwd=str(ROOT), timeout=60,
                         env=dict(os.environ))
    assert "RC 2" in out.stdout, out.stdout + out.stderr  # ncclSystemError
    assert "Init failed" in out.stderr
    os.environ.pop("MINI_NCCL_CONNECT_RETRIES")


def test_public_headers_compile_as_c_and_cpp_and_match_the_library(lib, tmp_path):
    """include/mini_nccl_api.h and include/mini_nccl_ops.h are self-contained in C and in C++, and every
    function they declare is exported by the library."""
    import re
    import shutil
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    cuda_inc = "/usr/local/cuda/include"
    if not (Path(cuda_inc) / "cuda_runtime.h").exists() or shutil.which("gcc") is None:
        pytest.skip("needs gcc and the CUDA headers")
    src = tmp_path / "hdr.c"
    src.write_text('#include "mini_nccl_api.h"\n#include "mini_nccl_ops.h"\nint main(void) { return 0; }\n')
    for cc, extra in (("gcc", []), ("g++", ["-x", "c++"])):
        r = subprocess.run([cc, "-fsyntax-only", "-Wall", "-Werror", *extra, f"-I{root / 'include'}", f"-I{cuda_inc}", str(src)],
                           capture_output=True, text=True)
        assert r.returncode == 0, r.stderr
    declared = set()
    for name in ("mini_nccl_api.h", "mini_nccl_ops.h"):
        text = (root / "include" / name).read_text()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        declared |= set(re.findall(r"\b((?:nccl|mnccl)[A-Za-z0-9]+)\s*\(", text))
    assert {"ncclAllReduce", "ncclCommInitRank", "mncclGemmBf16", "mncclSwiGluBf16"} <= declared
    missing = [f for f in sorted(declared) if not hasattr(lib, f)]
    assert not missing, f"declared but not exported: {missing}"
