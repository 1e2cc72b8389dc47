"""Worker bodies for the multi-process tests.  Each rank is its own Python process
(`python tests/mp_workers.py <fn> <rank> <nranks> <json kwargs>`), prints one line
`RESULT <json>` and exits 0; `run_ranks` starts them and collects the lines."""
from __future__ import annotations

import json
import os
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def run_ranks(fn: str, nranks: int, kwargs: dict | None = None, env: dict | None = None, timeout: float = 180.0,
              per_rank_env: dict | None = None, expect_rc=None):
    """Start `nranks` processes; return the list of result dicts ordered by rank."""
    base = dict(os.environ)
    base.update({k: str(v) for k, v in (env or {}).items()})
    base["PYTHONPATH"] = str(ROOT) + os.pathsep + base.get("PYTHONPATH", "")
    procs = []
    for r in range(nranks):
        e = dict(base)
        for k, v in (per_rank_env or {}).get(r, {}).items():
            e[k] = str(v)
        procs.append(subprocess.Popen([sys.executable, str(Path(__file__)), fn, str(r), str(nranks), json.dumps(kwargs or {})],
                                      env=e, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    deadline = time.time() + timeout
    outs = []
    for r, p in enumerate(procs):
        try:
            o, err = p.communicate(timeout=max(1.0, deadline - time.time()))
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            o, err = p.communicate()
            raise AssertionError(f"rank {r} timed out\nstdout:\n{o}\nstderr:\n{err[-4000:]}")
        outs.append((p.returncode, o, err))
    results = []
    for r, (rc, o, err) in enumerate(outs):
        want = 0 if expect_rc is None else expect_rc.get(r, 0)
        line = [l for l in o.splitlines() if l.startswith("RESULT ")]
        if rc != want or not line:
            raise AssertionError(f"rank {r} exited {rc} (wanted {want})\nstdout:\n{o[-3000:]}\nstderr:\n{err[-6000:]}")
        d = json.loads(line[-1][7:])
        d["_stderr"] = err
        results.append(d)
    return results


# --------------------------------------------------------------------------- helpers

def _np_inputs(dtype, count, n, op, seed=1234):
    from mini_nccl_b200.utils import oracle as O

    return [O.make_input(dtype, count, r, seed=seed, op=op) for r in range(n)]


def _bits_equal(a, b):
    import numpy as np

    return a.size == b.size and np.array_equal(a.view(np.uint8), b.view(np.uint8))


# --------------------------------------------------------------------------- CPU: ring over the soft transport

def cpu_ring(rank, n, kw):
    """AllReduce through the C ABI on host buffers (no GPU): the network data plane."""
    import ctypes as C

    import numpy as np

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib
    from mini_nccl_b200.utils import oracle as O

    init_rank = -1 if kw.get("hera") else rank
    comm = mn.Communicator(n, init_rank, kw.get("ip", "127.0.0.1"))
    rank = comm.rank
    n = comm.size
    res = {"rank": rank, "size": n, "cases": 0, "max_err": 0.0}
    for case in kw["cases"]:
        dtype, op, count = case["dtype"], case["op"], case["count"]
        ins = _np_inputs(dtype, count, n, op, seed=case.get("seed", 1234))
        x = ins[rank].copy()
        if case.get("in_place"):
            out = x
        else:
            out = np.zeros_like(x)
        for _ in range(case.get("repeat", 1)):
            if case.get("in_place"):
                x[:] = ins[rank]
            rc = mn.lib().ncclAllReduce(x.ctypes.data, out.ctypes.data, count, dtype, op, comm.handle, None)
            assert rc == 0, f"ncclAllReduce returned {rc}"
        want = O.oracle_allreduce(ins, dtype, op)
        if dtype == _lib.FLOAT32 and op == _lib.SUM:
            bad = C.c_size_t()
            ok = mn.lib().mnccl_verify_f32(out.ctypes.data, want.ctypes.data, count, 1e-5, C.byref(bad))
            assert ok == 0, f"AVX2 verifier: mismatch at {bad.value}: {out[bad.value]} vs {want[bad.value]}"
        if dtype in O.FLOAT_TYPES:
            # The ring adds in ring order, the oracle in rank order: compare with a tolerance.
            err = float(np.abs(O.to_float64(out, dtype) - O.to_float64(want, dtype)).max()) if count else 0.0
            tol = {_lib.FLOAT32: 1e-5, _lib.FLOAT64: 1e-12, _lib.FLOAT16: 0.02, _lib.BFLOAT16: 0.1}[dtype] * (4 if op == _lib.PROD else 1)
            assert err <= tol, f"{O.DTYPE_NAMES[dtype]} {O.OP_NAMES[op]} count {count}: err {err}"
            res["max_err"] = max(res["max_err"], err)
        else:
            assert _bits_equal(out, want), f"{O.DTYPE_NAMES[dtype]} {O.OP_NAMES[op]} count {count}: integer mismatch"
        res["cases"] += 1
    res["stats"] = comm.stats()
    comm.destroy()
    return res


def cpu_ring_fault(rank, n, kw):
    """A dropped flag write (host-side fault) must end in a bounded error, not a hang."""
    import numpy as np

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib

    comm = mn.Communicator(n, rank, "127.0.0.1")
    x = np.ones(kw.get("count", 1 << 16), np.float32)
    t0 = time.time()
    rc = mn.lib().ncclAllReduce(x.ctypes.data, x.ctypes.data, x.size, _lib.FLOAT32, _lib.SUM, comm.handle, None)
    dt = time.time() - t0
    err = comm.async_error() if rc != 0 else 0
    # after a failure the communicator stays failed (sticky), and destroy does not hang
    rc2 = mn.lib().ncclAllReduce(x.ctypes.data, x.ctypes.data, x.size, _lib.FLOAT32, _lib.SUM, comm.handle, None) if rc != 0 else 0
    comm.abort()
    comm.destroy()
    return {"rank": rank, "rc": rc, "rc2": rc2, "seconds": dt, "async": err}


# --------------------------------------------------------------------------- GPU: real multi-process data plane

def gpu_battery(rank, n, kw):
    import ctypes as C

    import numpy as np
    import torch

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib
    from mini_nccl_b200.utils import oracle as O

    torch.cuda.set_device(rank % torch.cuda.device_count())
    init_rank = -1 if kw.get("hera") else rank
    comm = mn.Communicator(n, init_rank, "127.0.0.1")
    rank, n = comm.rank, comm.size
    stats0 = comm.stats()
    res = {"rank": rank, "nvls": bool(stats0["nvls"]), "provider": stats0["symmetric_provider"], "plane": stats0["plane"],
           "cases": 0, "algos": {}}
    assert stats0["plane"] == "nvlink", stats0

    def T(np_arr):
        return torch.from_numpy(np_arr.view(np.uint8).copy()).cuda()

    tdt = {_lib.FLOAT32: torch.float32, _lib.BFLOAT16: torch.bfloat16, _lib.FLOAT16: torch.float16, _lib.FLOAT64: torch.float64,
           _lib.INT32: torch.int32, _lib.INT64: torch.int64, _lib.INT8: torch.int8, _lib.UINT8: torch.uint8}
    algos = ["ll", "oneshot", "twoshot", "auto"] + (["nvls"] if res["nvls"] else [])
    sym_cap = 8 << 20
    sym = comm.empty(sym_cap, torch.uint8)
    for algo in algos:
        for dtype, op, count in [(_lib.FLOAT32, _lib.SUM, 2048), (_lib.FLOAT32, _lib.SUM, 100003), (_lib.BFLOAT16, _lib.SUM, 65536 + 8),
                                 (_lib.BFLOAT16, _lib.AVG, 1 << 20), (_lib.FLOAT32, _lib.MAX, 5000), (_lib.INT32, _lib.SUM, 4097),
                                 (_lib.FLOAT16, _lib.SUM, 12345), (_lib.FLOAT64, _lib.PROD, 999), (_lib.INT8, _lib.MIN, 333)]:
            esz = _lib.DTYPE_SIZES[dtype]
            if algo == "ll" and count * esz > 64 * 1024:
                continue
            nvls_ok = dtype in (_lib.FLOAT32, _lib.BFLOAT16, _lib.FLOAT16) and op in (_lib.SUM, _lib.AVG)
            ins = _np_inputs(dtype, count, n, op)
            want = O.oracle_allreduce(ins, dtype, op)
            for where in ("plain", "symmetric"):
                if where == "plain":
                    buf = T(ins[rank])
                    out = torch.zeros_like(buf)
                else:
                    buf = sym[:count * esz]
                    buf.copy_(T(ins[rank]))
                    out = buf
                rc = mn.lib().mncclAllReduceEx(buf.data_ptr(), dtype, out.data_ptr(), dtype, dtype, count, op, 1.0,
                                               {"auto": 0, "ll": 1, "oneshot": 2, "twoshot": 3, "nvls": 4}[algo], comm.handle,
                                               torch.cuda.current_stream().cuda_stream)
                assert rc == 0, f"{algo} {O.DTYPE_NAMES[dtype]} {O.OP_NAMES[op]} {count} {where}: rc {rc}"
                torch.cuda.synchronize()
                got = out.cpu().numpy().view(O.NP_DTYPES[dtype])
                if algo in ("nvls", "auto") and nvls_ok and res["nvls"]:
                    # the switch defines the summation order: tolerance instead of bits
                    err = float(np.abs(O.to_float64(got, dtype) - O.to_float64(want, dtype)).max())
                    assert err <= O.tolerance(dtype, n), f"{algo} {O.DTYPE_NAMES[dtype]} {count} {where}: err {err}"
                else:
                    assert _bits_equal(got, want), f"{algo} {O.DTYPE_NAMES[dtype]} {O.OP_NAMES[op]} {count} {where}: mismatch"
                res["cases"] += 1
                comm.barrier()
    # large message on ordinary buffers: the chunk pipeline (copy-in / collective / copy-out overlapped)
    count = (16 << 20) + 12345
    ins = _np_inputs(_lib.FLOAT32, count, n, _lib.SUM)
    want = O.oracle_allreduce(ins, _lib.FLOAT32, _lib.AVG)
    big = torch.from_numpy(ins[rank]).cuda()
    big_out = torch.zeros_like(big)
    comm.all_reduce(big, "avg", out=big_out)
    torch.cuda.synchronize()
    err = float(np.abs(big_out.cpu().numpy() - want).max())
    assert err <= (1e-5 * n if res["nvls"] else 0.0), f"pipelined AllReduce: err {err}"
    # ... which is, by rank count and what the machine offers: the two-shot kernel with lazy direct access,
    # the pipelined kernel, or copy kernels on side streams around the collective
    st_big = comm.stats()
    assert (st_big["pipelined_calls"] >= 1 or st_big["algo"].get("pipe", 0) >= 1 or st_big["auto_map"]["exports"] >= 1), st_big
    gp = torch.cuda.CUDAGraph()
    sp = torch.cuda.Stream()
    sp.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(sp):
        with torch.cuda.graph(gp, stream=sp):
            comm.all_reduce(big, "avg", out=big_out)
    torch.cuda.current_stream().wait_stream(sp)
    big_out.zero_()
    gp.replay()
    gp.replay()
    torch.cuda.synchronize()
    err = float(np.abs(big_out.cpu().numpy() - want).max())
    assert err <= (1e-5 * n if res["nvls"] else 0.0), f"pipelined AllReduce in a graph: err {err}"
    del gp, big, big_out
    # an ordinary tensor registered through CUDA IPC is used in place by the peer-to-peer kernels
    count = 1 << 20
    ins = _np_inputs(_lib.FLOAT32, count, n, _lib.SUM)
    want = O.oracle_allreduce(ins, _lib.FLOAT32, _lib.SUM)
    reg = torch.from_numpy(ins[rank]).cuda()
    comm.register(reg)
    zc0 = comm.stats()["zero_copy_in"]
    comm.all_reduce(reg, "sum", algo="twoshot")
    torch.cuda.synchronize()
    assert np.array_equal(reg.cpu().numpy(), want), "registered buffer: mismatch"
    st = comm.stats()
    assert st["zero_copy_in"] == zc0 + 1 and st["ipc_cache"]["open"] >= n - 1   # lazy direct access may hold mappings too
    view = reg[1024:1024 + 4096]            # a view inside the same allocation hits the handle cache
    comm.register(view)
    assert comm.stats()["ipc_cache"]["hits"] >= 0
    comm.deregister(reg)
    # A registered buffer that is freed and whose range is allocated again: the library notices the new
    # allocation (driver buffer id) and refuses the call instead of reducing through stale peer mappings.
    rt = C.CDLL("libcudart.so.12")
    pa, pb = C.c_void_p(), C.c_void_p()
    assert rt.cudaMalloc(C.byref(pa), C.c_size_t(4 << 20)) == 0
    _lib.check(_lib.lib().mncclCommRegister(comm.handle, pa, 4 << 20), "mncclCommRegister")
    assert rt.cudaFree(pa) == 0
    assert rt.cudaMalloc(C.byref(pb), C.c_size_t(4 << 20)) == 0
    same = torch.tensor([1.0 if pb.value == pa.value else 0.0], device="cuda")
    comm.all_reduce(same, "min")
    res["stale_registration_checked"] = bool(same.item() == 1.0)
    if res["stale_registration_checked"]:      # every rank got its old range back
        rc = _lib.lib().mncclAllReduce(pb, pb, 1 << 20, _lib.FLOAT32, _lib.SUM, comm.handle, None)
        assert rc == _lib.INVALID_USAGE, f"stale registration not refused: rc {rc}"
        assert comm.stats()["stale_registrations"] >= 1
    _lib.check(_lib.lib().mncclCommDeregister(comm.handle, pa), "mncclCommDeregister")
    assert rt.cudaFree(pb) == 0
    x = torch.ones(1 << 20, device="cuda")
    comm.all_reduce(x, "sum")                   # the communicator is as usable as before
    torch.cuda.synchronize()
    assert torch.all(x == float(n)).item()
    # NVLS on exactly representable data is bit-exact whatever the order
    if res["nvls"]:
        count = 1 << 18
        x = torch.full((count,), float(rank + 1), device="cuda")
        s = comm.empty(count, torch.float32)
        s.copy_(x)
        comm.all_reduce(s, "sum", algo="nvls")
        torch.cuda.synchronize()
        assert torch.all(s == float(n * (n + 1) // 2)).item()
        comm.free(s)
    # fused cast + scale
    count = 300001
    ins = _np_inputs(_lib.FLOAT32, count, n, _lib.SUM)
    want = O.oracle_allreduce(ins, _lib.FLOAT32, _lib.SUM, wire_dtype=_lib.BFLOAT16, out_dtype=_lib.FLOAT32, scale=0.5)
    src = torch.from_numpy(ins[rank]).cuda()
    dst = torch.zeros(count, device="cuda")
    comm.all_reduce(src, "sum", out=dst, scale=0.5, wire_dtype=torch.bfloat16, algo="twoshot")
    torch.cuda.synchronize()
    assert np.array_equal(dst.cpu().numpy(), want), "fused fp32->bf16->fp32 mismatch"
    # reduce-scatter / all-gather
    per = 50003
    ins = _np_inputs(_lib.FLOAT32, per * n, n, _lib.SUM)
    want = O.oracle_allreduce(ins, _lib.FLOAT32, _lib.SUM)
    src = torch.from_numpy(ins[rank]).cuda()
    rs = torch.zeros(per, device="cuda")
    comm.reduce_scatter(src, rs)
    torch.cuda.synchronize()
    got_rs = rs.cpu().numpy()
    if res["nvls"]:  # large ReduceScatter may go through the switch, which picks the summation order
        assert float(np.abs(got_rs - want[rank * per:(rank + 1) * per]).max()) <= 1e-5 * n, "reduce_scatter mismatch"
    else:
        assert np.array_equal(got_rs, want[rank * per:(rank + 1) * per]), "reduce_scatter mismatch"
    ag = torch.zeros(per * n, device="cuda")
    comm.all_gather(rs, ag)
    torch.cuda.synchronize()
    # AllGather moves bits: every rank must hold exactly what each owner computed
    assert np.array_equal(ag.cpu().numpy()[rank * per:(rank + 1) * per], got_rs), "all_gather: own shard changed"
    assert float(np.abs(ag.cpu().numpy() - want).max()) <= 1e-5 * n, "all_gather mismatch"
    chk = ag.clone()
    comm.all_reduce(chk, "max")
    torch.cuda.synchronize()
    assert torch.equal(chk, ag), "all_gather results differ between ranks"
    # pinned host buffers, as the reference's programs use
    hx = torch.from_numpy(_np_inputs(_lib.FLOAT32, 1 << 20, n, _lib.SUM)[rank]).pin_memory()
    hy = torch.zeros(1 << 20).pin_memory()
    rc = mn.lib().mncclAllReduce(hx.data_ptr(), hy.data_ptr(), 1 << 20, _lib.FLOAT32, _lib.SUM, comm.handle, None)
    assert rc == 0
    torch.cuda.synchronize()
    want = O.oracle_allreduce(_np_inputs(_lib.FLOAT32, 1 << 20, n, _lib.SUM), _lib.FLOAT32, _lib.SUM)
    if res["nvls"]:
        assert float(np.abs(hy.numpy() - want).max()) <= 1e-5 * n
    else:
        assert np.array_equal(hy.numpy(), want), "pinned host buffers mismatch"
    # larger pinned buffers are moved by the copy engines in chunks that overlap the collective:
    # several chunks, a count that is no multiple of anything, in place
    cnt = (6 << 20) + 1000
    big = _np_inputs(_lib.FLOAT32, cnt, n, _lib.SUM)
    hb = torch.from_numpy(big[rank].copy()).pin_memory()
    before = comm.stats()["pipelined_calls"]
    comm.all_reduce(hb, "sum")
    torch.cuda.synchronize()
    want = O.oracle_allreduce(big, _lib.FLOAT32, _lib.SUM)
    if res["nvls"]:
        assert float(np.abs(hb.numpy() - want).max()) <= 1e-5 * n, "pinned host pipeline mismatch"
    else:
        assert np.array_equal(hb.numpy(), want), "pinned host pipeline mismatch"
    assert comm.stats()["pipelined_calls"] == before + 1, "large pinned buffers must take the copy-engine pipeline"
    # device in, pinned host out, fused average
    dv = torch.from_numpy(big[rank].copy()).cuda()
    ho = torch.zeros(cnt).pin_memory()
    comm.all_reduce(dv, "avg", out=ho)
    torch.cuda.synchronize()
    assert float(np.abs(ho.numpy() - want / n).max()) <= 2e-6 * n, "device -> pinned host average mismatch"
    # CUDA graph: capture 50 AllReduces of 64 KB bf16, replay 20 times
    g_in = comm.empty(32768, torch.bfloat16)
    ones = torch.ones(32768, dtype=torch.bfloat16, device="cuda")
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        g_in.copy_(ones)
        comm.all_reduce(g_in, "avg")
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            for _ in range(50):
                comm.all_reduce(g_in, "avg")
    torch.cuda.current_stream().wait_stream(s)
    for _ in range(20):
        g.replay()
    torch.cuda.synchronize()
    assert torch.all(g_in == 1.0).item(), "graph replay changed the average of ones"
    assert comm.async_error() == 0
    res["stats"] = comm.stats()
    res["algo_8k"] = comm.query_algo(8192)
    res["algo_1m"] = comm.query_algo(1 << 20)
    res["algo_256m"] = comm.query_algo(256 << 20, registered=True)
    del g
    comm.free(g_in)
    comm.free(sym)
    comm.destroy()
    return res


def gpu_stall(rank, n, kw):
    """1000 AllReduces of 64 KB bf16 in CUDA graphs; one rank stops launching at iteration
    `stall_at` (a host-made stall).  Every rank must see an error within the bound."""
    import torch

    import mini_nccl_b200 as mn

    torch.cuda.set_device(rank % torch.cuda.device_count())
    init_rank = -1 if kw.get("hera") else rank
    comm = mn.Communicator(n, init_rank, "127.0.0.1")
    rank = comm.rank
    buf = comm.empty(32768, torch.bfloat16)
    buf.fill_(1.0)
    per_graph = 10
    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        comm.all_reduce(buf, "avg")
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            for _ in range(per_graph):
                comm.all_reduce(buf, "avg")
    torch.cuda.synchronize()
    comm.barrier()
    stall_at, victim = kw["stall_at"], kw["victim"]
    t_fail, it_fail = None, None
    t0 = time.time()
    for it in range(0, kw["iters"], per_graph):
        if rank == victim and it == stall_at:
            # the stalled rank simply stops launching; it polls the error state instead
            while comm.async_error() in (0, 7) and time.time() - t0 < 60:  # 7: its own earlier kernels still run
                time.sleep(0.01)
        if comm.async_error() not in (0, 7):
            t_fail, it_fail = time.time(), it
            break
        with torch.cuda.stream(s):
            g.replay()
        if it % 100 == 0:
            s.synchronize()
    if t_fail is None:
        s.synchronize()
        if comm.async_error() not in (0, 7):
            t_fail, it_fail = time.time(), kw["iters"]
    torch.cuda.synchronize()  # every kernel has returned: nothing is left spinning
    t_sync = time.time()
    err = comm.async_error()
    rc = 0
    try:
        comm.all_reduce(buf, "avg")
    except mn.MiniNcclError as e:
        rc = e.code
    stats = comm.stats()
    comm.destroy()
    return {"rank": rank, "async": err, "rc_after": rc, "it_fail": it_fail, "sync_seconds": t_sync - t0, "stats": stats}


def gpu_tp(rank, n, kw):
    """Fused tensor-parallel kernels across real GPUs against a PyTorch fp32 reference."""
    import torch

    import mini_nccl_b200 as mn
    from mini_nccl_b200.ops import AllGatherGemm, GemmReduceScatter, gemm_status

    torch.cuda.set_device(rank % torch.cuda.device_count())
    comm = mn.Communicator(n, rank, "127.0.0.1")
    M, N, K = kw.get("M", 1024), kw.get("N", 1024), kw.get("K", 512)
    per = M // n
    rs = GemmReduceScatter(comm, M, N)
    ag = AllGatherGemm(comm, M, K, n_comm_ctas=kw.get("n_comm", 16))
    worst = 0.0
    for it in range(kw.get("iters", 4)):
        # every rank can rebuild every rank's operands from the seeds
        def operands(r):
            g = torch.Generator(device="cuda").manual_seed(1000 * it + r)
            a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
            b = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
            x = torch.randn(per, K, generator=g, device="cuda").to(torch.bfloat16)
            return a, b, x
        mine = operands(rank)
        # GEMM -> reduce-scatter: rows of this rank of sum_r A_r B_r^T
        ref = torch.zeros(per, N, device="cuda")
        for r in range(n):
            a, b, _ = operands(r)
            ref += a[rank * per:(rank + 1) * per].float() @ b.float().t()
        out = rs(mine[0], mine[1])
        torch.cuda.synchronize()
        assert gemm_status() == 0, "a bounded wait ran out in GEMM->reduce-scatter"
        err = (out.float() - ref).abs().max().item() / ref.abs().max().item()
        assert err < 1e-2, f"gemm_rs it {it}: rel err {err}"
        worst = max(worst, err)
        # all-gather -> GEMM: stack of every rank's x times my b
        xs = torch.cat([operands(r)[2] for r in range(n)])
        ref2 = xs.float() @ mine[1].float().t()
        ag.local_shard.copy_(mine[2])
        c = ag(mine[1])
        torch.cuda.synchronize()
        assert gemm_status() == 0, "a bounded wait ran out in all-gather->GEMM"
        assert torch.equal(ag.gather, xs), f"ag_gemm it {it}: gathered rows differ"
        err2 = (c.float() - ref2).abs().max().item() / ref2.abs().max().item()
        assert err2 < 1e-2, f"ag_gemm it {it}: rel err {err2}"
        worst = max(worst, err2)
    # bit for bit against the host restatement on integer-valued operands (rank order, roundings)
    from mini_nccl_b200.utils import verify

    res = verify.check_fused_gemm(comm, n, rank, M=M, N=N, K=K)
    assert res["failed"] == 0, res["failures"]
    comm.barrier()
    comm.destroy()
    return {"rank": rank, "worst": worst, "oracle_cases": res["cases"], "rs_in_switch": bool(rs.in_switch)}


def gpu_tp_stall(rank, n, kw):
    """GEMM -> reduce-scatter under the communicator's failure model: after two good steps the victim
    stops launching (a stall made on the host, between steps, none of its kernels in flight); the other
    ranks' kernels wait for its tiles, the watchdog sets the abort word after the configured bound, the
    kernels return, the communicator reports an error and takes no more work."""
    import torch

    import mini_nccl_b200 as mn
    from mini_nccl_b200.ops import GemmReduceScatter, gemm_status

    torch.cuda.set_device(rank % torch.cuda.device_count())
    comm = mn.Communicator(n, rank, "127.0.0.1")
    M, N, K = 1024, 1024, 256
    rs = GemmReduceScatter(comm, M, N)
    g = torch.Generator(device="cuda").manual_seed(rank)
    a = torch.randn(M, K, generator=g, device="cuda").to(torch.bfloat16)
    b = torch.randn(N, K, generator=g, device="cuda").to(torch.bfloat16)
    for _ in range(2):
        rs(a, b)
    torch.cuda.synchronize()
    comm.barrier()
    t0 = time.time()
    raised = 0
    if rank == kw["victim"]:
        while comm.async_error() in (0, 7) and time.time() - t0 < 60:  # learns of the failure on the host (shared abort page)
            time.sleep(0.01)
    else:
        rs(a, b)                      # waits for the victim's tiles that never come
        torch.cuda.synchronize()      # ... and returns within the bound
    waited = time.time() - t0
    err = comm.async_error()
    try:
        rs(a, b)
    except mn.MiniNcclError as e:
        raised = e.code
    status = gemm_status()
    stats = comm.stats()
    comm.destroy()
    return {"rank": rank, "async": err, "raised": raised, "waited": waited, "gemm_status": status, "stats": stats}


def gpu_shared(rank, n, kw):
    """Every rank on GPU 0 (the reference benchmark's layout): the host-synchronised plane.  Device and
    pinned-host buffers, several types and operators, a message larger than the staging buffer, in
    place and out of place, all bit for bit against the rank-ordered host oracle."""
    import numpy as np
    import torch

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib
    from mini_nccl_b200.utils import oracle as O

    torch.cuda.set_device(0)
    comm = mn.Communicator(n, rank, "127.0.0.1")
    stats0 = comm.stats()
    cases = 0
    tdt = {_lib.FLOAT32: torch.float32, _lib.BFLOAT16: torch.bfloat16, _lib.INT32: torch.int32, _lib.FLOAT64: torch.float64}
    for code, op, opname, count in ((_lib.FLOAT32, _lib.SUM, "sum", 1 << 20), (_lib.FLOAT32, _lib.SUM, "sum", 5),
                                    (_lib.BFLOAT16, _lib.SUM, "sum", (1 << 19) + 3), (_lib.INT32, _lib.MAX, "max", 70001),
                                    (_lib.FLOAT64, _lib.PROD, "prod", 4099), (_lib.FLOAT32, _lib.AVG, "avg", 300001),
                                    (_lib.FLOAT32, _lib.SUM, "sum", kw.get("big", (5 << 20) + 7))):
        ins = [O.make_input(code, count, r, op=op) for r in range(n)]
        want = O.oracle_allreduce(ins, code, op)
        for where in ("device", "pinned"):
            raw = torch.from_numpy(ins[rank].view(np.int16) if code == _lib.BFLOAT16 else ins[rank])
            src = raw.view(tdt[code]) if code == _lib.BFLOAT16 else raw
            if where == "device":
                x = src.cuda()
                y = torch.empty_like(x)
            else:
                x = src.clone().pin_memory()
                y = torch.empty_like(x).pin_memory()
            comm.all_reduce(x, opname, out=y)
            torch.cuda.synchronize()
            got = y.cpu()
            got = got.view(torch.int16).numpy().view(np.uint16) if code == _lib.BFLOAT16 else got.numpy()
            assert np.array_equal(got, want), f"{where} {O.DTYPE_NAMES[code]} {opname} {count}: {int(np.count_nonzero(got != want))} differ"
            cases += 1
        # in place on the device
        x = (torch.from_numpy(ins[rank].view(np.int16)).view(torch.bfloat16) if code == _lib.BFLOAT16 else torch.from_numpy(ins[rank])).cuda()
        comm.all_reduce(x, opname)
        torch.cuda.synchronize()
        got = x.cpu()
        got = got.view(torch.int16).numpy().view(np.uint16) if code == _lib.BFLOAT16 else got.numpy()
        assert np.array_equal(got, want)
        cases += 1
    # a rough rate on device buffers (host clock: the call is host-synchronous)
    big = torch.ones(16 << 20, device="cuda")
    comm.all_reduce(big, "sum")
    t0 = time.time()
    for _ in range(5):
        comm.all_reduce(big, "sum")
    dt = (time.time() - t0) / 5
    stats = comm.stats()
    comm.destroy()
    return {"rank": rank, "cases": cases, "plane": stats0["plane"], "hostsync": stats["algo"].get("hostsync", 0),
            "algbw_GBps": (64 << 20) / dt / 1e9}


def gpu_auto_map(rank, n, kw):
    """Ordinary torch tensors through the peer-to-peer two-shot AllReduce: the first call stages, later
    calls on the same allocations run on the user buffers directly once every rank has mapped them.
    Every result is compared bit for bit with the rank-ordered host oracle."""
    import numpy as np
    import torch

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib
    from mini_nccl_b200.utils import oracle as O

    torch.cuda.set_device(rank % torch.cuda.device_count())
    comm = mn.Communicator(n, rank, "127.0.0.1")
    want_direct = kw.get("expect_direct", True)
    out = {"rank": rank, "cases": 0, "steps": []}

    def run(count, dtype_code, tdt, in_place, seed, buf=None):
        ins = [O.make_input(dtype_code, count, r, seed=seed, dist="normal") for r in range(n)]
        want = O.oracle_allreduce(ins, dtype_code, _lib.SUM, scale=1.0)
        if buf is None:
            buf = (torch.empty(count, dtype=tdt, device="cuda"), None if in_place else torch.empty(count, dtype=tdt, device="cuda"))
        src, dst = buf
        raw = ins[rank].view(np.int16) if dtype_code == _lib.BFLOAT16 else ins[rank]
        (src.view(torch.int16) if dtype_code == _lib.BFLOAT16 else src).copy_(torch.from_numpy(raw.copy()))
        comm.all_reduce(src, "sum", out=dst, algo="twoshot")
        torch.cuda.synchronize()
        res = dst if dst is not None else src
        got = (res.view(torch.int16) if dtype_code == _lib.BFLOAT16 else res).cpu().numpy()
        got = got.view(np.uint16) if dtype_code == _lib.BFLOAT16 else got
        assert np.array_equal(got, want), f"rank {rank}: count {count} seed {seed}: {int(np.count_nonzero(got != want))} elements differ"
        out["cases"] += 1
        comm.barrier()   # the next call finds this call's exports of every rank
        out["steps"].append(comm.stats()["auto_map"]["direct_calls"])
        return buf

    # the same buffers again and again (a training loop's gradient bucket), 24 MB fp32, out of place
    big = None
    for it in range(4):
        big = run((6 << 20) + 3, _lib.FLOAT32, torch.float32, False, 100 + it, big)
    direct_after_reuse = comm.stats()["auto_map"]["direct_calls"]
    # in place, bf16, a message above the stream pipeline's threshold
    loop = None
    for it in range(3):
        loop = run(40 << 20, _lib.BFLOAT16, torch.bfloat16, True, 200 + it, loop)
    # a buffer that was never seen: staged on its first call, and still right
    run(1 << 20 | 1, _lib.FLOAT32, torch.float32, False, 300)
    st = comm.stats()
    out.update({"auto_map": st["auto_map"], "pipelined_calls": st["pipelined_calls"], "direct_after_reuse": direct_after_reuse,
                "algo": st["algo"]})
    if want_direct:
        assert st["auto_map"]["exports"] >= 2 and st["auto_map"]["imports"] >= 2 * (n - 1), st["auto_map"]
        assert direct_after_reuse >= 2, out["steps"]
    else:
        assert st["auto_map"]["direct_calls"] == 0 and st["auto_map"]["exports"] == 0
    comm.destroy()
    return out


FUNCS = {f.__name__: f for f in (cpu_ring, cpu_ring_fault, gpu_battery, gpu_stall, gpu_tp, gpu_tp_stall, gpu_shared, gpu_auto_map)}

if __name__ == "__main__":
    fn, rank, n, kw = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), json.loads(sys.argv[4])
    out = FUNCS[fn](rank, n, kw)
    print("RESULT " + json.dumps(out))
    sys.stdout.flush()
