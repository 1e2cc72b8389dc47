"""Device kernels on ONE GPU: N virtual ranks inside one cooperative launch.

Covers every algorithm that runs on peer loads / stores (LL, one-shot,
two-shot, ReduceScatter, AllGather) for all data types and operators, odd
sizes, unaligned pointers, staged multi-pass and zero-copy paths, fused casts,
back-to-back calls (epochs, inbox parity) and the bounded wait.  Results are
compared bit for bit with the rank-ordered host oracle and, with a tolerance,
with a plain PyTorch fp32 reference.
"""
import ctypes as C

import numpy as np
import pytest

from mini_nccl_b200 import _lib
from mini_nccl_b200.utils import oracle as O

pytestmark = pytest.mark.gpu

ALL_DTYPES = [_lib.INT8, _lib.UINT8, _lib.INT32, _lib.UINT32, _lib.INT64, _lib.UINT64, _lib.FLOAT16, _lib.FLOAT32,
              _lib.FLOAT64, _lib.BFLOAT16]
ALL_OPS = [_lib.SUM, _lib.PROD, _lib.MAX, _lib.MIN, _lib.AVG]
ALGOS = {"ll": _lib.ALGO_LL, "oneshot": _lib.ALGO_ONESHOT, "twoshot": _lib.ALGO_TWOSHOT, "pipe": 7}


class World:
    def __init__(self, lib, n, staging=0):
        import torch

        self.torch = torch
        self.lib, self.n = lib, n
        self.h = C.c_void_p()
        rc = lib.mncclEmuCreate(n, staging, C.byref(self.h))
        assert rc == 0, rc

    def close(self):
        if self.h:
            self.lib.mncclEmuDestroy(self.h)
            self.h = C.c_void_p()

    def upload(self, arr, offset_elems=0):
        """Host array -> device tensor of raw bytes (optionally shifted to break alignment)."""
        t = self.torch
        raw = np.ascontiguousarray(arr).view(np.uint8)
        pad = offset_elems * arr.dtype.itemsize
        buf = t.empty(raw.size + pad + 64, dtype=t.uint8, device="cuda")
        view = buf[pad:pad + raw.size]
        view.copy_(t.from_numpy(raw.copy()))
        return buf, view

    def run(self, mode, sends, recvs, count, in_t, wire_t, out_t, op, scale=1.0, algo=0, nblocks=0):
        sp = (C.c_void_p * self.n)(*[s.data_ptr() for s in sends])
        rp = (C.c_void_p * self.n)(*[r.data_ptr() for r in recvs])
        rc = self.lib.mncclEmuCollective(self.h, mode, sp, rp, count, in_t, wire_t, out_t, op, scale, algo, nblocks, None)
        assert rc == 0, f"emulated collective failed: {rc}"
        self.torch.cuda.synchronize()
        st = (C.c_uint32 * self.n)()
        assert self.lib.mncclEmuStatus(self.h, st, None) == 0
        assert list(st) == [0] * self.n, f"device status {list(st)}"

    def last_plan(self):
        a, b = C.c_int(), C.c_int()
        self.lib.mncclEmuLastPlan(self.h, C.byref(a), C.byref(b))
        return _lib.ALGO_NAMES[a.value], b.value


def download(view, np_dtype):
    return view.cpu().numpy().view(np_dtype).copy()


def check_allreduce(world, count, dtype, op, algo, in_place=False, misalign=0, wire=None, out_t=None, scale=1.0,
                    nblocks=0, seed=1234):
    n = world.n
    wire = dtype if wire is None else wire
    out_t = dtype if out_t is None else out_t
    ins = [O.make_input(dtype, count, r, seed=seed, op=op) for r in range(n)]
    keep, sends, recvs = [], [], []
    for r in range(n):
        b, v = world.upload(ins[r], offset_elems=misalign)
        keep.append(b)
        sends.append(v)
        if in_place:
            recvs.append(v)
        else:
            out_bytes = count * _lib.DTYPE_SIZES[out_t]
            ob = world.torch.zeros(out_bytes + 128, dtype=world.torch.uint8, device="cuda")
            keep.append(ob)
            recvs.append(ob[misalign * _lib.DTYPE_SIZES[out_t]: misalign * _lib.DTYPE_SIZES[out_t] + out_bytes])
    world.run(0, sends, recvs, count, dtype, wire, out_t, op, scale=scale, algo=algo, nblocks=nblocks)
    want = O.oracle_allreduce(ins, dtype, op, wire_dtype=wire, out_dtype=out_t, scale=scale)
    ref = O.torch_fp32_reference(ins, dtype, op, scale=scale)
    for r in range(n):
        got = download(recvs[r], O.NP_DTYPES[out_t])
        assert got.size == count
        bad = np.nonzero(got.view(np.uint8).reshape(count, -1) != want.view(np.uint8).reshape(count, -1))[0]
        assert bad.size == 0, (f"rank {r}: first mismatch at {bad[0]} got {got[bad[0]]} want {want[bad[0]]} "
                               f"({O.DTYPE_NAMES[dtype]} {O.OP_NAMES[op]} n={n} count={count} plan={world.last_plan()})")
        if wire == dtype and out_t == dtype and op != _lib.PROD:
            err = np.abs(O.to_float64(got, out_t) - ref).max() if count else 0.0
            assert err <= O.tolerance(dtype, n) + 1e-30, f"vs torch fp32 reference: {err}"


@pytest.fixture(scope="module")
def worlds(lib):
    made = {}

    def get(n, staging=0):
        key = (n, staging)
        if key not in made:
            made[key] = World(lib, n, staging)
        return made[key]

    yield get
    for w in made.values():
        w.close()


@pytest.mark.parametrize("n", [2, 4, 8])
@pytest.mark.parametrize("algo", ["ll", "oneshot", "twoshot"])
def test_allreduce_fp32_sum_sizes(worlds, n, algo):
    w = worlds(n)
    for count in (1, 3, 7, 255, 1024, 4099, 65536 + 5):
        if algo == "ll" and count * 4 > 64 * 1024:
            continue
        check_allreduce(w, count, _lib.FLOAT32, _lib.SUM, ALGOS[algo])
        assert w.last_plan()[0] == algo


@pytest.mark.parametrize("dtype", ALL_DTYPES)
@pytest.mark.parametrize("algo", ["ll", "oneshot", "twoshot"])
def test_allreduce_every_dtype_and_op(worlds, dtype, algo):
    w = worlds(4)
    for op in ALL_OPS:
        check_allreduce(w, 1000 + 13, dtype, op, ALGOS[algo])


@pytest.mark.parametrize("algo", ["ll", "oneshot", "twoshot"])
def test_allreduce_in_place_and_unaligned(worlds, algo):
    w = worlds(4)
    check_allreduce(w, 5001, _lib.FLOAT32, _lib.SUM, ALGOS[algo], in_place=True)
    check_allreduce(w, 5001, _lib.BFLOAT16, _lib.SUM, ALGOS[algo], misalign=1)
    check_allreduce(w, 777, _lib.INT8, _lib.MAX, ALGOS[algo], misalign=3, in_place=True)
    check_allreduce(w, 2049, _lib.FLOAT64, _lib.SUM, ALGOS[algo], misalign=1)


@pytest.mark.parametrize("n", [2, 8])
def test_twoshot_multi_pass_staging(worlds, n):
    # 1 MiB of staging forces several passes over a 12 MB message.
    w = worlds(n, staging=1 << 20)
    check_allreduce(w, 3 * 1024 * 1024 + 17, _lib.FLOAT32, _lib.SUM, _lib.ALGO_TWOSHOT)
    check_allreduce(w, 3 * 1024 * 1024 + 17, _lib.BFLOAT16, _lib.AVG, _lib.ALGO_TWOSHOT, in_place=True)


def test_auto_selection_large(worlds):
    w = worlds(8)
    check_allreduce(w, 8 * 1024 * 1024, _lib.BFLOAT16, _lib.SUM, _lib.ALGO_AUTO)
    assert w.last_plan()[0] == "twoshot"  # NVLS needs a real multicast mapping


@pytest.mark.parametrize("algo", ["ll", "oneshot", "twoshot"])
def test_fused_cast_and_scale(worlds, algo):
    w = worlds(4)
    a = ALGOS[algo]
    check_allreduce(w, 4096 + 3, _lib.FLOAT32, _lib.SUM, a, wire=_lib.BFLOAT16, out_t=_lib.FLOAT32, scale=0.25)
    check_allreduce(w, 4096 + 3, _lib.FLOAT32, _lib.AVG, a, wire=_lib.BFLOAT16, out_t=_lib.BFLOAT16)
    check_allreduce(w, 4096 + 3, _lib.BFLOAT16, _lib.SUM, a, wire=_lib.BFLOAT16, out_t=_lib.FLOAT32, scale=0.125)
    check_allreduce(w, 4096 + 3, _lib.BFLOAT16, _lib.AVG, a, scale=2.0)


def test_back_to_back_mixed_algorithms(worlds):
    # Epochs, LL sequence numbers and inbox parity must survive any interleaving.
    w = worlds(4)
    seq = ["ll", "ll", "oneshot", "ll", "twoshot", "oneshot", "oneshot", "twoshot", "twoshot", "ll", "oneshot"]
    for i, algo in enumerate(seq * 2):
        check_allreduce(w, 3000 + i, _lib.FLOAT32, _lib.SUM, ALGOS[algo], seed=100 + i)


def test_zero_copy_symmetric_buffers(worlds, lib):
    import torch

    w = worlds(4)
    count = 1 << 20
    ptrs = (C.c_void_p * 4)()
    assert lib.mncclEmuAlloc(w.h, count * 4, ptrs) == 0
    ins = [O.make_input(_lib.FLOAT32, count, r) for r in range(4)]

    from mini_nccl_b200.utils.interop import tensor_from_ptr

    bufs = [tensor_from_ptr(ptrs[r], count * 4, torch.float32) for r in range(4)]
    for r in range(4):
        bufs[r].copy_(torch.from_numpy(ins[r]))
    w.run(0, bufs, bufs, count, _lib.FLOAT32, _lib.FLOAT32, _lib.FLOAT32, _lib.SUM, algo=_lib.ALGO_TWOSHOT)
    assert w.last_plan()[0] == "twoshot"
    want = O.oracle_allreduce(ins, _lib.FLOAT32, _lib.SUM)
    for r in range(4):
        assert np.array_equal(bufs[r].cpu().numpy(), want)
    # out of place: symmetric input, ordinary output
    for r in range(4):
        bufs[r].copy_(torch.from_numpy(ins[r]))
    outs = [torch.zeros(count, dtype=torch.float32, device="cuda") for _ in range(4)]
    w.run(0, bufs, outs, count, _lib.FLOAT32, _lib.FLOAT32, _lib.FLOAT32, _lib.AVG, algo=_lib.ALGO_TWOSHOT)
    want = O.oracle_allreduce(ins, _lib.FLOAT32, _lib.AVG)
    for r in range(4):
        assert np.array_equal(outs[r].cpu().numpy(), want)


@pytest.mark.parametrize("dtype", [_lib.FLOAT32, _lib.BFLOAT16, _lib.INT32])
def test_reduce_scatter_and_all_gather(worlds, dtype):
    import torch

    n = 4
    w = worlds(n)
    for per_rank in (1024, 1001, 5):
        ins = [O.make_input(dtype, per_rank * n, r) for r in range(n)]
        keep = [w.upload(a) for a in ins]
        outs = [torch.zeros(per_rank * _lib.DTYPE_SIZES[dtype], dtype=torch.uint8, device="cuda") for _ in range(n)]
        w.run(1, [k[1] for k in keep], outs, per_rank, dtype, dtype, dtype, _lib.SUM, algo=_lib.ALGO_TWOSHOT)
        want = O.oracle_allreduce(ins, dtype, _lib.SUM)
        for r in range(n):
            got = download(outs[r], O.NP_DTYPES[dtype])
            assert np.array_equal(got, want[r * per_rank:(r + 1) * per_rank]), f"reduce_scatter rank {r} per_rank {per_rank}"
        # all-gather of the first per_rank elements of every rank
        shards = [a[:per_rank].copy() for a in ins]
        keep2 = [w.upload(a) for a in shards]
        outs2 = [torch.zeros(per_rank * n * _lib.DTYPE_SIZES[dtype], dtype=torch.uint8, device="cuda") for _ in range(n)]
        w.run(2, [k[1] for k in keep2], outs2, per_rank, dtype, dtype, dtype, _lib.SUM, algo=_lib.ALGO_TWOSHOT)
        cat = np.concatenate(shards)
        for r in range(n):
            assert np.array_equal(download(outs2[r], O.NP_DTYPES[dtype]), cat), f"all_gather rank {r} per_rank {per_rank}"


def test_bounded_wait_returns_timeout_and_abort(lib):
    st, us = C.c_uint32(), C.c_uint32()
    assert lib.mncclProbeBoundedWait(20_000_000, 0, C.byref(st), C.byref(us)) == 0
    assert st.value == 1, "a wait on a flag nobody sets must time out"
    assert 15_000 <= us.value <= 2_000_000
    assert lib.mncclProbeBoundedWait(5_000_000_000, 1, C.byref(st), C.byref(us)) == 0
    assert st.value == 2, "a set abort word must end the wait"
    assert us.value < 1_000_000


def test_missing_rank_fails_bounded(lib):
    # One virtual rank takes no part: the others' waits run out after the
    # configured budget, the kernel returns and reports a status; the context
    # stays usable.
    import torch

    w = World(lib, 4)
    try:
        assert lib.mncclEmuSetTimeoutNs(w.h, 30_000_000) == 0
        assert lib.mncclEmuSetDeaf(w.h, 2, 1) == 0
        ins = [torch.ones(1024, device="cuda") for _ in range(4)]
        sp = (C.c_void_p * 4)(*[t.data_ptr() for t in ins])
        rc = lib.mncclEmuCollective(w.h, 0, sp, sp, 1024, _lib.FLOAT32, _lib.FLOAT32, _lib.FLOAT32, _lib.SUM, 1.0,
                                    _lib.ALGO_ONESHOT, 0, None)
        assert rc == 0
        torch.cuda.synchronize()
        st, det = (C.c_uint32 * 4)(), (C.c_uint32 * 4)()
        assert lib.mncclEmuStatus(w.h, st, det) == 0
        assert st[2] == 0 and all(st[r] == 1 for r in (0, 1, 3)), list(st)
        assert all((det[r] & 0xFFFF) == 2 for r in (0, 1, 3)), "the failure names the silent peer"
    finally:
        w.close()
    x = torch.ones(16, device="cuda")
    assert float((x + 1).sum()) == 32.0


# ------------------------------------------------------------------ pipelined kernel (ordinary buffers)
@pytest.mark.parametrize("n", [2, 4, 8])
def test_pipe_kernel_wraps_slot_ring(worlds, lib, n):
    """Copy-in, reduce and copy-out blocks of ONE kernel, chunk by chunk: with 64 KB chunks a
    message of a few MB runs many times around the ring of 64 staging slots, and the second and
    third call continue the chunk numbering where the one before stopped."""
    w = worlds(n, 64 << 20)
    assert lib.mncclEmuSetPipeChunk(w.h, 64 << 10) == 0
    try:
        for count in (3 * 1024 * 1024 + 77, 1 << 20, 16 * 1024 + 3, 5):
            check_allreduce(w, count, _lib.FLOAT32, _lib.SUM, ALGOS["pipe"], seed=count)
            assert w.last_plan()[0] == "pipe"
        check_allreduce(w, 2 * 1024 * 1024 + 1, _lib.BFLOAT16, _lib.SUM, ALGOS["pipe"], scale=1.0 / n)
        check_allreduce(w, 700001, _lib.FLOAT32, _lib.SUM, ALGOS["pipe"], misalign=1)          # unaligned user buffers
        check_allreduce(w, 1 << 20, _lib.FLOAT32, _lib.SUM, ALGOS["pipe"], wire=_lib.BFLOAT16)  # fp32 -> bf16 wire -> fp32
        check_allreduce(w, 1 << 20, _lib.FLOAT32, _lib.SUM, ALGOS["pipe"], wire=_lib.BFLOAT16, out_t=_lib.BFLOAT16)
        check_allreduce(w, 300001, _lib.INT32, _lib.MAX, ALGOS["pipe"])
        check_allreduce(w, 300001, _lib.FLOAT64, _lib.PROD, ALGOS["pipe"])
        check_allreduce(w, 1 << 20, _lib.FLOAT32, _lib.SUM, ALGOS["pipe"], in_place=True)
    finally:
        lib.mncclEmuSetPipeChunk(w.h, 0)


def test_pipe_kernel_few_blocks(worlds, lib):
    """Three blocks (one per role) are the smallest grid; the roles must still hand over correctly."""
    w = worlds(2, 64 << 20)
    assert lib.mncclEmuSetPipeChunk(w.h, 256 << 10) == 0
    try:
        for nb in (3, 4, 5, 7):
            check_allreduce(w, 2 * 1024 * 1024 + 9, _lib.FLOAT32, _lib.SUM, ALGOS["pipe"], nblocks=nb, seed=nb)
    finally:
        lib.mncclEmuSetPipeChunk(w.h, 0)


def test_ll_calls_with_changing_block_counts(worlds):
    """LL inbox slots are addressed by unit offset, the flag comes from ONE sequence per communicator:
    calls that split the same units over 1, 2, 3 ... blocks, with fresh data every time, must never
    accept a packet of an earlier call."""
    w = worlds(4, 0)
    count = 3000                      # 12 KB fp32: a few blocks' worth of 8-byte units
    for i, nb in enumerate([1, 2, 1, 3, 2, 4, 1, 4, 3, 1, 2, 2]):
        check_allreduce(w, count, _lib.FLOAT32, _lib.SUM, ALGOS["ll"], nblocks=nb, seed=1000 + i)
        assert w.last_plan() == ("ll", nb)


@pytest.mark.parametrize("n", [2, 4, 8])
def test_lazy_direct_access_agrees_inside_the_kernel(lib, n):
    """The two-shot kernel on ordinary buffers goes direct only when EVERY rank has EVERY rank's buffers
    in its table; one missing row on one rank keeps all ranks on the staged path.  Bit-exact either way,
    in place and out of place, with a message of several staging passes."""
    w = World(lib, n, staging=1 << 20)
    try:
        direct = (C.c_uint32 * n)()
        full = [1] * (n * n)
        partial = list(full)
        partial[1 * n + 0] = 0            # rank 1 has not mapped rank 0's buffers yet
        seen = 0
        for mapped, goes_direct in ((partial, False), (full, True), (partial, False), (full, True)):
            assert lib.mncclEmuSetAutoMap(w.h, (C.c_int * (n * n))(*mapped)) == 0
            for dtype, count, in_place in ((_lib.FLOAT32, (3 << 20) + 5, False), (_lib.BFLOAT16, 1 << 20, True),
                                           (_lib.INT32, 70001, False)):
                op = _lib.MAX if dtype == _lib.INT32 else _lib.SUM
                check_allreduce(w, count, dtype, op, ALGOS["twoshot"], in_place=in_place, seed=77 + seen)
                assert w.last_plan()[0] == "twoshot"
                assert lib.mncclEmuDirectCalls(w.h, direct) == 0
                seen += 1 if goes_direct else 0
                assert list(direct) == [seen] * n, (list(direct), seen, mapped == full)
        # buffers that are not 16-byte aligned stay staged although every table is complete
        check_allreduce(w, 40000, _lib.FLOAT32, _lib.SUM, ALGOS["twoshot"], misalign=1)
        assert lib.mncclEmuDirectCalls(w.h, direct) == 0 and list(direct) == [seen] * n
        assert lib.mncclEmuSetAutoMap(w.h, None) == 0
    finally:
        w.close()
