"""The network data plane on its own, without a GPU: N processes on this host run the
slice / window / signal-batch ring over the one-sided soft provider (TCP on loopback) through the
C ABI, with the method of the reference's benchmark (reference: tests/perf_test.cpp:60-65,87-99,
140-143): fp32 sum, out of place, 5 warm-up + 20 timed iterations per size, host clock,
algBW = bytes / time, busBW = algBW * 2(n-1)/n; time is the maximum over ranks.

  python benchmarks/net_plane_bench.py --ranks 2 --sizes-mib 1 4 16 64 128
"""
from __future__ import annotations

import argparse
import json
import multiprocessing as mp
import os
import socket
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, n, port, sizes, iters, warmup, q, transport):
    os.environ["MINI_NCCL_TRANSPORT"] = transport
    os.environ["MINI_NCCL_BOOTSTRAP_PORT"] = str(port)
    import numpy as np

    import mini_nccl_b200 as mn
    from mini_nccl_b200 import _lib

    comm = mn.Communicator(n, rank, "127.0.0.1")
    rows = []
    for nbytes in sizes:
        count = nbytes // 4
        rng = np.random.default_rng(1234 + rank)
        x = rng.uniform(-1.0, 1.0, count).astype(np.float32)
        y = np.zeros_like(x)

        def once():
            rc = mn.lib().ncclAllReduce(x.ctypes.data, y.ctypes.data, count, _lib.FLOAT32, _lib.SUM, comm.handle, None)
            assert rc == 0, rc

        for _ in range(warmup):
            once()
        comm.barrier()
        t0 = time.perf_counter()
        for _ in range(iters):
            once()
        dt = (time.perf_counter() - t0) / iters
        rows.append((nbytes, dt, float(y[:8].sum())))
    q.put((rank, rows))
    comm.destroy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ranks", type=int, default=2)
    ap.add_argument("--sizes-mib", type=float, nargs="+", default=[1, 4, 16, 64, 128])
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--transport", default="soft", choices=["soft", "verbs"],
                    help="verbs needs a library built with libibverbs (or the test stand-in: MINI_NCCL_LIB)")
    args = ap.parse_args()
    sizes = [int(s * (1 << 20)) for s in args.sizes_mib]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, args.ranks, port, sizes, args.iters, args.warmup, q, args.transport)) for r in range(args.ranks)]
    for p in procs:
        p.start()
    got = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    n = args.ranks
    print(f"{'Size(B)':>12} {'Time(us)':>12} {'AlgBW(GB/s)':>12} {'BusBW(GB/s)':>12}")
    out = []
    for i, nbytes in enumerate(sizes):
        t = max(rows[i][1] for _, rows in got)
        alg = nbytes / t / 1e9
        bus = alg * 2 * (n - 1) / n
        print(f"{nbytes:>12} {t * 1e6:>12.1f} {alg:>12.3f} {bus:>12.3f}")
        out.append({"bytes": nbytes, "us": round(t * 1e6, 1), "algbw_GBps": round(alg, 3), "busbw_GBps": round(bus, 3)})
    print(json.dumps({"ranks": n, "provider": args.transport, "rows": out}))


if __name__ == "__main__":
    main()
