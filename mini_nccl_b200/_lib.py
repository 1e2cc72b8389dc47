"""ctypes binding to libmini_nccl.so.

The Python side binds to the ``mnccl*`` entry points, never to the ``nccl*``
names: a PyTorch process already has the real NCCL loaded, whose
``ncclCommInitRank`` has a different signature (the reference re-exports NCCL's
symbol names with its own signature, reference: include/mini_nccl_api.h:57).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

_HERE = Path(__file__).resolve().parent
_LIB = None

# ncclResult_t
SUCCESS, UNHANDLED_CUDA_ERROR, SYSTEM_ERROR, INTERNAL_ERROR, INVALID_ARGUMENT, INVALID_USAGE, REMOTE_ERROR, IN_PROGRESS = range(8)
# ncclDataType_t
INT8, UINT8, INT32, UINT32, INT64, UINT64, FLOAT16, FLOAT32, FLOAT64, BFLOAT16 = range(10)
# ncclRedOp_t
SUM, PROD, MAX, MIN, AVG = range(5)
# mncclAlgo_t
ALGO_AUTO, ALGO_LL, ALGO_ONESHOT, ALGO_TWOSHOT, ALGO_NVLS, ALGO_RING = range(6)
ALGO_NAMES = {0: "auto", 1: "ll", 2: "oneshot", 3: "twoshot", 4: "nvls", 5: "ring", 6: "local", 7: "pipe"}
DTYPE_SIZES = {INT8: 1, UINT8: 1, INT32: 4, UINT32: 4, INT64: 8, UINT64: 8, FLOAT16: 2, FLOAT32: 4, FLOAT64: 8, BFLOAT16: 2}


class MiniNcclError(RuntimeError):
    def __init__(self, code: int, where: str):
        self.code = code
        msg = lib().mncclGetErrorString(code).decode()
        super().__init__(f"{where}: {msg} (ncclResult_t {code})")


def lib_file() -> Path:
    """The shared object to load; MINI_NCCL_LIB overrides the in-tree default (used by the tests
    to load the variant built against the stand-in verbs implementation)."""
    override = os.environ.get("MINI_NCCL_LIB")
    return Path(override) if override else _HERE / "lib" / "libmini_nccl.so"


def lib() -> C.CDLL:
    """Load (building first if the shared object is missing) and type the library."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_file()
    if not path.exists():
        if os.environ.get("MINI_NCCL_NO_BUILD") == "1":
            raise RuntimeError(f"{path} is missing and MINI_NCCL_NO_BUILD=1")
        from . import build as _build
        _build.build()
    L = C.CDLL(str(path), mode=C.RTLD_LOCAL)
    vp, sz, i32, u32, u64, dbl = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_uint64, C.c_double
    P = C.POINTER

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype = res
        f.argtypes = list(args)

    sig("mncclGetErrorString", C.c_char_p, i32)
    sig("mncclCommInitRank", i32, P(vp), i32, i32, C.c_char_p)
    sig("mncclCommDestroy", i32, vp)
    sig("mncclCommUserRank", i32, vp, P(i32))
    sig("mncclCommCount", i32, vp, P(i32))
    sig("mncclAllReduce", i32, vp, vp, sz, i32, i32, vp, vp)
    sig("mncclAllReduceEx", i32, vp, i32, vp, i32, i32, sz, i32, dbl, i32, vp, vp)
    sig("mncclReduceScatter", i32, vp, vp, sz, i32, i32, vp, vp)
    sig("mncclAllGather", i32, vp, vp, sz, i32, vp, vp)
    sig("mncclMemAlloc", i32, vp, sz, P(vp))
    sig("mncclMemFree", i32, vp, vp)
    sig("mncclMemPeerPointers", i32, vp, vp, P(vp), P(vp))
    sig("mncclCommRegister", i32, vp, vp, sz)
    sig("mncclCommDeregister", i32, vp, vp)
    sig("mncclBarrier", i32, vp)
    sig("mncclCommAbort", i32, vp)
    sig("mncclCommGetAsyncError", i32, vp, P(i32))
    sig("mncclCommStats", i32, vp, C.c_char_p, sz)
    sig("mncclCommQueryAlgo", i32, vp, sz, i32, i32, i32, P(i32))
    sig("mncclCommDeviceHandle", i32, vp, vp, sz, P(sz))
    sig("mncclCommSetTuning", i32, vp, i32, i32)
    sig("mncclCommSetKnob", i32, vp, C.c_char_p, C.c_longlong)
    sig("mncclVersion", C.c_uint)
    # reference-compatible names (exported for C users; typed here for the ABI tests)
    sig("ncclGetErrorString", C.c_char_p, i32)
    sig("ncclCommInitRank", i32, P(vp), i32, i32, C.c_char_p)
    sig("ncclCommDestroy", i32, vp)
    sig("ncclCommUserRank", i32, vp, P(i32))
    sig("ncclCommCount", i32, vp, P(i32))
    sig("ncclAllReduce", i32, vp, vp, sz, i32, i32, vp, vp)
    # sm_100a GEMM (optional translation unit)
    if hasattr(L, "mncclGemmBf16"):
        sig("mncclGemmBf16", i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, vp)
        sig("mncclGemmStatus", i32, P(u32))
        if hasattr(L, "mncclGemmSetPairMode"):
            sig("mncclGemmSetPairMode", None, i32)
        if hasattr(L, "mncclGemmPlan"):
            sig("mncclGemmPlan", None, i32, i32, i32, i32, C.POINTER(C.c_int), C.POINTER(C.c_int))
    if hasattr(L, "mncclSwiGluBf16"):
        sig("mncclSwiGluBf16", i32, vp, vp, i32, i32, C.c_long, C.c_long, vp)
    if hasattr(L, "mncclGemmReduceScatterBf16"):
        sig("mncclGemmRsStageBytes", sz, i32, i32, i32)
        sig("mncclGemmRsFlagWords", sz, i32, i32, i32)
        sig("mncclAgGemmReadyWords", sz, i32)
        sig("mncclAgGemmBarWords", sz, i32, i32)
        sig("mncclGemmReduceScatterBf16", i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, P(vp), P(vp), vp, vp)
        sig("mncclAllGatherGemmBf16", i32, P(vp), vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, P(vp), P(vp), vp, i32, vp)
        sig("mncclAllGatherGemmSwiGluBf16", i32, P(vp), vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, P(vp), P(vp), vp, i32, vp)
        sig("mncclGemmReduceScatterBf16Comm", i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, P(vp), P(vp), vp, C.c_char_p, sz, vp)
        sig("mncclGemmReduceScatterBf16Switch", i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, P(vp), P(vp), vp, vp, i32,
            C.c_char_p, sz, vp)
        sig("mncclAllGatherGemmBf16Comm", i32, P(vp), vp, vp, i32, i32, i32, i32, i32, i32, i32, i32, P(vp), P(vp), vp, i32, i32,
            C.c_char_p, sz, vp)
        sig("mncclGemmProbeFlagWait", i32, u64, i32, P(u32), P(u32), P(u32))
    # emulation + probes
    sig("mncclEmuCreate", i32, i32, sz, P(vp))
    sig("mncclEmuDestroy", i32, vp)
    sig("mncclEmuAlloc", i32, vp, sz, P(vp))
    sig("mncclEmuSetTimeoutNs", i32, vp, u64)
    sig("mncclEmuSetDeaf", i32, vp, i32, i32)
    sig("mncclEmuSetPipeChunk", i32, vp, sz)
    sig("mncclEmuCollective", i32, vp, i32, P(vp), P(vp), sz, i32, i32, i32, i32, dbl, i32, i32, vp)
    sig("mncclEmuStatus", i32, vp, P(u32), P(u32))
    if hasattr(L, "mncclEmuSetAutoMap"):
        sig("mncclEmuSetAutoMap", i32, vp, P(C.c_int))
        sig("mncclEmuDirectCalls", i32, vp, P(u32))
    sig("mncclEmuLastPlan", i32, vp, P(i32), P(i32))
    sig("mncclProbeBoundedWait", i32, u64, i32, P(u32), P(u32))
    # host oracle (csrc/ref/oracle_api.cc)
    sig("mnccl_oracle_allreduce", i32, i32, i32, i32, i32, i32, P(vp), vp, sz, dbl)
    sig("mnccl_verify_f32", i32, vp, vp, sz, C.c_float, P(sz))
    sig("mnccl_verify_const_f32", i32, vp, C.c_float, sz, C.c_float, P(sz))
    sig("mnccl_sum_f32", None, vp, vp, vp, sz)
    sig("mnccl_cpu_has_avx2", i32)
    sig("mnccl_float_to_bf16", C.c_uint16, C.c_float)
    sig("mnccl_float_to_half", C.c_uint16, C.c_float)
    sig("mnccl_bf16_to_float", C.c_float, C.c_uint16)
    sig("mnccl_half_to_float", C.c_float, C.c_uint16)
    # Entry points for the test-suite live in a library of their own (libmini_nccl_testhooks.so, the same
    # objects plus csrc/testing/hooks.cc); when it is present they are attached to this handle under
    # their names, so tests call them like any other function.  The product library exports none of them.
    hooks_path = path.parent / "libmini_nccl_testhooks.so"
    if hooks_path.exists():
        H = C.CDLL(str(hooks_path), mode=C.RTLD_LOCAL)

        def hsig(name, res, *args):
            f = getattr(H, name)
            f.restype = res
            f.argtypes = list(args)
            setattr(L, name, f)

        hsig("mnccl_test_config", i32, C.c_char_p, C.c_char_p, sz)
        hsig("mnccl_test_tuning_text", i32, C.c_char_p, i32, C.c_char_p, sz)
        hsig("mnccl_test_pipeline_chunks", i32, sz, sz, sz, sz, i32, P(sz), i32)
        hsig("mnccl_test_soft_reject", i32, i32, i32)
        hsig("mnccl_test_spsc", i32, i32, i32)
        hsig("mnccl_test_request_pool", i32, i32)
        hsig("mnccl_test_reg_cache", i32)
        hsig("mnccl_test_select_nic", i32, C.c_char_p, C.c_char_p, P(i32))
        hsig("mnccl_test_parse_cpu_list", i32, C.c_char_p, P(i32), i32)
        hsig("mnccl_test_numa", i32, C.c_char_p, C.c_char_p, P(i32), P(i32))
        hsig("mnccl_test_plan", i32, i32, i32, u64, i32, i32, i32, i32, i32, i32, i32, i32, u64, P(i32), P(i32), P(u64), P(u64), P(i32), P(i32))
        hsig("mnccl_test_watchdog", i32, i32, i32)
        hsig("mnccl_test_fdpass", i32, C.c_char_p)
        hsig("mnccl_hera_master_start", vp, i32, i32, i32)
        hsig("mnccl_hera_master_port", i32, vp)
        hsig("mnccl_hera_master_registered", i32, vp)
        hsig("mnccl_hera_master_abort_sent", i32, vp)
        hsig("mnccl_hera_master_worker", i32, vp, i32, P(i32), P(i32), C.c_char_p, C.c_char_p, P(i32))
        hsig("mnccl_hera_master_stop", None, vp)
        hsig("mnccl_hera_worker_register", vp, C.c_char_p, i32, P(i32), P(i32), C.c_char_p)
        hsig("mnccl_hera_worker_topology", i32, vp, P(i32), P(i32), C.c_char_p)
        hsig("mnccl_hera_worker_start_agent", i32, vp, i32, i32)
        hsig("mnccl_hera_worker_abort_seen", i32, i32)
        hsig("mnccl_hera_worker_send_abort", i32, vp, C.c_uint)
        hsig("mnccl_hera_worker_set_state", None, vp, C.c_uint)
        hsig("mnccl_hera_worker_free", None, vp)
    _LIB = L
    return L


def hooks_lib() -> C.CDLL:
    """The test-suite's own copy of the library (libmini_nccl_testhooks.so): the same objects plus the
    entry points of csrc/testing/hooks.cc.  It has its own static state, so a test that needs a hook to
    act on library state (the allocation-free entry point's scratch) makes ALL its calls through it."""
    path = lib_file().parent / "libmini_nccl_testhooks.so"
    if not path.exists():
        raise RuntimeError(f"{path} is missing (built by mini_nccl_b200.build)")
    return C.CDLL(str(path), mode=C.RTLD_LOCAL)


def check(code: int, where: str) -> None:
    if code != SUCCESS:
        raise MiniNcclError(code, where)
