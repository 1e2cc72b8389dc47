"""The checked build of the collective kernels (libmini_nccl_devcheck.so, -DMNCCL_DEVICE_CHECKS=1): every
staging access is tested against its area's size and alignment first; a bad one is recorded in the status
word and skipped -- it never traps and the access never happens.  The bad accesses are made on purpose by
telling the kernels a staging size SMALLER than the memory the emulated world really owns, so that even an
access a check missed would stay inside owned memory: nothing here can fault."""
import ctypes as C
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

LIB = Path(__file__).resolve().parent.parent / "mini_nccl_b200" / "lib" / "libmini_nccl_devcheck.so"


def _load():
    if not LIB.exists():
        from mini_nccl_b200 import build

        build.build_devcheck_variant()
    L = C.CDLL(str(LIB), mode=C.RTLD_LOCAL)
    vp, sz, i32, u32, dbl = C.c_void_p, C.c_size_t, C.c_int, C.c_uint32, C.c_double
    L.mncclEmuCreate.argtypes = [i32, sz, C.POINTER(vp)]
    L.mncclEmuDestroy.argtypes = [vp]
    L.mncclEmuClaimStageBytes.argtypes = [vp, sz]
    L.mncclEmuCollective.argtypes = [vp, i32, C.POINTER(vp), C.POINTER(vp), sz, i32, i32, i32, i32, dbl, i32, i32, vp]
    L.mncclEmuStatus.argtypes = [vp, C.POINTER(u32), C.POINTER(u32)]
    return L


def _run(L, world, n, ins, outs, count):
    sp = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
    rp = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
    FLOAT32, SUM, TWOSHOT = 7, 0, 3
    assert L.mncclEmuCollective(world, 0, sp, rp, count, FLOAT32, FLOAT32, FLOAT32, SUM, 1.0, TWOSHOT, 0, None) == 0
    st, det = (C.c_uint32 * n)(), (C.c_uint32 * n)()
    assert L.mncclEmuStatus(world, st, det) == 0
    return list(st), list(det)


def test_checked_build_records_and_skips_accesses_beyond_the_claimed_staging():
    import torch

    L = _load()
    assert L.mncclBuiltWithDeviceChecks() == 1
    n, count = 2, 1 << 20                       # 4 MB per rank through 4 MB of staging: one pass, offsets up to 4 MB
    ins = [torch.full((count,), float(r + 1), device="cuda") for r in range(n)]
    outs = [torch.zeros(count, device="cuda") for _ in range(n)]
    # a world told the truth: status 0 and the right sums
    w = C.c_void_p()
    assert L.mncclEmuCreate(n, 4 << 20, C.byref(w)) == 0
    try:
        st, _ = _run(L, w, n, ins, outs, count)
        assert st == [0, 0]
        assert all(torch.equal(o, torch.full_like(o, 3.0)) for o in outs)
    finally:
        L.mncclEmuDestroy(w)
    # a world whose kernels are told that only the first MB of each staging area exists
    w = C.c_void_p()
    assert L.mncclEmuCreate(n, 4 << 20, C.byref(w)) == 0
    try:
        assert L.mncclEmuClaimStageBytes(w, 1 << 20) == 0
        for o in outs:
            o.zero_()
        st, det = _run(L, w, n, ins, outs, count)
        assert st == [3, 3], f"status {st}: the checks must record kDevBadIndex"
        assert all(d >= (1 << 20) // 16 for d in det), "detail is the offending offset in 16-byte units"
        torch.cuda.synchronize()
        # what lay inside the claimed megabyte was still reduced; nothing was written where an access was skipped
        head = (1 << 20) // 4 // n               # elements of each shard that fit the claimed area
        got = outs[0].cpu().numpy()
        assert np.all(got[:head] == 3.0)
        assert np.count_nonzero(got) < count
    finally:
        L.mncclEmuDestroy(w)


def test_product_library_is_built_without_the_checks(lib):
    lib.mncclBuiltWithDeviceChecks.restype = C.c_int
    assert lib.mncclBuiltWithDeviceChecks() == 0
