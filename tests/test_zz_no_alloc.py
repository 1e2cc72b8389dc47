"""The allocation-free AllReduce over buffers of one GPU, called through its exported C symbol
and compared with the entry point that allocates its scratch (the emulated one-shot AllReduce).

Collected last on purpose (pytest orders files by name): a run that stops at the first failure
has then already run every other test.  It shares no state with them: it must pass alone in a
fresh process and after the whole suite, which is why it loads the library itself and makes
two calls in a row on the same static scratch (the second one sees what the first left)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _lib():
    from mini_nccl_b200 import _lib as L

    lib = L.lib()
    fn = lib.mncclLocalAllReduceNoAlloc
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    lib.mncclNoAllocScratchBytes.restype = C.c_size_t
    return L, lib


def _reference(L, lib, torch, inputs, count, dtype, op):
    """The existing entry point: emulated one-shot AllReduce with cudaMalloc'ed scratch."""
    n = len(inputs)
    world = C.c_void_p()
    assert lib.mncclEmuCreate(n, 0, C.byref(world)) == 0
    try:
        bufs = [t.clone() for t in inputs]
        ptrs = (C.c_void_p * n)(*[b.data_ptr() for b in bufs])
        assert lib.mncclEmuCollective(world, 0, ptrs, ptrs, count, dtype, dtype, dtype, op, 1.0, L.ALGO_ONESHOT, 0, None) == 0
        torch.cuda.synchronize()
        return [b.cpu() for b in bufs]
    finally:
        lib.mncclEmuDestroy(world)


def test_no_alloc_matches_allocating_entry_point_twice_in_a_row():
    import torch

    L, lib = _lib()
    assert 0 < lib.mncclNoAllocScratchBytes() <= 8 << 20, "the static scratch is meant to be modest"
    cases = [(4, 16384, L.FLOAT32, torch.float32, L.SUM), (3, 4099, L.BFLOAT16, torch.bfloat16, L.AVG),
             (2, 777, L.INT32, torch.int32, L.MAX), (4, 32768, L.FLOAT16, torch.float16, L.SUM)]
    for n, count, code, tdt, op in cases:
        for call in range(2):  # two calls in a row share the static scratch
            g = torch.Generator(device="cuda").manual_seed(1234 + call)
            if tdt == torch.int32:
                ins = [torch.randint(-1000, 1000, (count,), generator=g, device="cuda", dtype=tdt) for _ in range(n)]
            else:
                ins = [torch.randn(count, generator=g, device="cuda").to(tdt) for _ in range(n)]
            want = _reference(L, lib, torch, ins, count, code, op)
            outs = [torch.zeros_like(t) for t in ins]
            sp = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
            rp = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
            rc = lib.mncclLocalAllReduceNoAlloc(sp, rp, n, count, code, op, None)
            assert rc == 0, f"rc {rc}"
            torch.cuda.synchronize()
            # both entry points run the same rank-ordered kernel body: the results are the same bits
            for r in range(n):
                assert torch.equal(outs[r].cpu(), want[r]), (n, count, tdt, op, call, r)
            st, det = C.c_uint(7), C.c_uint(7)
            assert lib.mncclNoAllocLastStatus(None, C.byref(st), C.byref(det)) == 0 and st.value == 0
            # in place works too
            sp2 = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
            assert lib.mncclLocalAllReduceNoAlloc(sp2, sp2, n, count, code, op, None) == 0
            torch.cuda.synchronize()
            assert all(torch.equal(ins[r].cpu(), outs[r].cpu()) for r in range(n))


def test_no_alloc_allocates_nothing_and_ignores_what_the_last_call_left():
    """Free device memory is the same before and after a call (the first call on the device may load the
    kernel, so the check is on a later one), and a call does not depend on the control words the one
    before it left behind: the scratch is dirtied with a direct copy between two calls."""
    import torch

    L, _ = _lib()
    # every call of this test goes through the test-suite's own copy of the library: the hook that
    # dirties the scratch acts on that copy's static array
    lib = L.hooks_lib()
    lib.mncclLocalAllReduceNoAlloc.restype = C.c_int
    lib.mncclLocalAllReduceNoAlloc.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    rt = C.CDLL("libcudart.so.12")
    n, count = 4, 8192
    ins = [torch.full((count,), float(r + 1), device="cuda") for r in range(n)]
    outs = [torch.zeros_like(t) for t in ins]
    sp = (C.c_void_p * n)(*[t.data_ptr() for t in ins])
    rp = (C.c_void_p * n)(*[t.data_ptr() for t in outs])
    assert lib.mncclLocalAllReduceNoAlloc(sp, rp, n, count, L.FLOAT32, L.SUM, None) == 0   # first call: set-up
    torch.cuda.synchronize()
    free0, total = C.c_size_t(), C.c_size_t()
    assert rt.cudaMemGetInfo(C.byref(free0), C.byref(total)) == 0
    for _ in range(3):
        assert lib.mncclLocalAllReduceNoAlloc(sp, rp, n, count, L.FLOAT32, L.SUM, None) == 0
    torch.cuda.synchronize()
    free1 = C.c_size_t()
    assert rt.cudaMemGetInfo(C.byref(free1), C.byref(total)) == 0
    assert free1.value == free0.value, "the call changed the amount of free device memory"
    assert all(torch.equal(o, torch.full_like(o, 10.0)) for o in outs)
    # leave garbage in the barrier words and the per-rank state (as an aborted call would), call again
    assert lib.mnccl_test_noalloc_dirty(0xA5) == 0
    for o in outs:
        o.zero_()
    assert lib.mncclLocalAllReduceNoAlloc(sp, rp, n, count, L.FLOAT32, L.SUM, None) == 0
    torch.cuda.synchronize()
    assert all(torch.equal(o, torch.full_like(o, 10.0)) for o in outs)
    st = C.c_uint(7)
    assert lib.mncclNoAllocLastStatus(None, C.byref(st), None) == 0 and st.value == 0


def test_no_alloc_rejects_what_exceeds_the_static_scratch():
    import torch

    L, lib = _lib()
    x = [torch.zeros(20000, device="cuda") for _ in range(5)]
    p5 = (C.c_void_p * 5)(*[t.data_ptr() for t in x])
    assert lib.mncclLocalAllReduceNoAlloc(p5, p5, 5, 16, L.FLOAT32, L.SUM, None) == L.INVALID_ARGUMENT   # too many buffers
    assert lib.mncclLocalAllReduceNoAlloc(p5, p5, 1, 16, L.FLOAT32, L.SUM, None) == L.INVALID_ARGUMENT   # nothing to reduce
    assert lib.mncclLocalAllReduceNoAlloc(p5, p5, 4, 16385, L.FLOAT32, L.SUM, None) == L.INVALID_ARGUMENT  # > 64 KiB each
    assert lib.mncclLocalAllReduceNoAlloc(p5, p5, 4, 16, L.FLOAT64, L.SUM, None) == L.INVALID_ARGUMENT   # unsupported type
    assert lib.mncclLocalAllReduceNoAlloc(None, p5, 4, 16, L.FLOAT32, L.SUM, None) == L.INVALID_ARGUMENT
    assert lib.mncclLocalAllReduceNoAlloc(p5, p5, 4, 0, L.FLOAT32, L.SUM, None) == 0                     # empty: nothing to do
    assert lib.mncclLocalAllReduceNoAlloc(p5, p5, 4, 16384, L.FLOAT32, L.SUM, None) == 0                  # exactly the maximum
    torch.cuda.synchronize()
