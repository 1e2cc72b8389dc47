"""AllReduce bandwidth / latency sweep: this library against NCCL on the same box.

Sizes double from 8 KB; fp32 and bf16 sum; inputs normal(0,1) seeded per rank;
every number is device-timed (CUDA events) and the maximum over ranks.  For each
size the library is timed on symmetric buffers (zero-copy) and on ordinary torch
tensors (staged), NCCL through torch.distributed on ordinary tensors.  Messages
smaller than the L2 are followed by an L2 flush kernel between iterations when
``flush`` is set (the quick mode used by bench.py reports back-to-back numbers
and says so).

Run stand-alone under torchrun:
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/sweep.py --out sweep.json
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _time_loop(fn, iters, warmup, world, repeats=1):
    """Milliseconds per call: `iters` back-to-back calls between two CUDA events on the current
    stream, after `warmup` calls and a barrier; the maximum over ranks; the MEDIAN of `repeats`
    such loops (a single short loop is exposed to one-off stalls of a shared machine, the best of
    several flatters)."""
    import torch
    import torch.distributed as dist

    from mini_nccl_b200.utils.timing import max_over_ranks

    for _ in range(warmup):
        fn()
    seen = []
    for _ in range(repeats):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            fn()
        e1.record()
        torch.cuda.synchronize()
        ms = max_over_ranks(e0.elapsed_time(e1) / iters)
        seen.append(ms)
    return sorted(seen)[(len(seen) - 1) // 2]


def nccl_registered_buffer(numel, dtype):
    """A tensor from NCCL's own allocator (ncclMemAlloc through ``torch.cuda.MemPool``), registered with the
    process group's communicator, so that NCCL can use it in place (and through the switch): the
    like-for-like partner of this library's symmetric buffers.  Returns (tensor, pool) or (None, reason)."""
    import torch
    import torch.distributed as dist

    try:
        backend = dist.group.WORLD._get_backend(torch.device("cuda"))
        pool = torch.cuda.MemPool(backend.mem_allocator)
        with torch.cuda.use_mem_pool(pool):
            t = torch.empty(numel, dtype=dtype, device="cuda")
        backend.register_mem_pool(pool)
        return t, pool
    except Exception as e:  # an older torch, an NCCL without the allocator, ...
        return None, f"{type(e).__name__}: {e}"[:120]


def run_sweep(comm, world, rank, max_bytes=1 << 30, min_bytes=8 << 10, quick=False, dtypes=("fp32", "bf16"),
              algos=("auto",), with_nccl=True, graphs=True, nccl_registered=False):
    import torch
    import torch.distributed as dist

    from mini_nccl_b200.utils.timing import bus_bandwidth_gbs

    rows = []
    sizes = []
    b = min_bytes
    while b <= max_bytes:
        sizes.append(b)
        b *= 2
    sym_cap = max(sizes)
    sym = {}
    for dt_name in dtypes:
        dt = torch.float32 if dt_name == "fp32" else torch.bfloat16
        esz = 4 if dt_name == "fp32" else 2
        if world > 1:
            sym[dt_name] = comm.empty(sym_cap // esz, dt)
        plain = torch.empty(sym_cap // esz, dtype=dt, device="cuda")
        reg, reg_pool = (None, None)
        if nccl_registered and with_nccl and world > 1:
            reg, reg_pool = nccl_registered_buffer(sym_cap // esz, dt)
        gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
        init = torch.randn(min(sym_cap // esz, 1 << 24), generator=gen, device="cuda").to(dt)
        for nbytes in sizes:
            n = nbytes // esz
            iters = 200 if nbytes <= (1 << 20) else (50 if nbytes <= (64 << 20) else 15)
            if quick:
                iters = max(5, iters // 3)
            warm = 5
            reps = 3
            row = {"bytes": nbytes, "dtype": dt_name}
            scale = 1.0 / world
            for algo in algos:
                key = "ours" if algo == "auto" else f"ours_{algo}"
                if world > 1:
                    t = sym[dt_name][:n]
                    t.copy_(init[:n] if n <= init.numel() else init.repeat((n + init.numel() - 1) // init.numel())[:n])
                    try:
                        ms = _time_loop(lambda: comm.all_reduce(t, "sum", scale=scale, algo=algo), iters, warm, world, reps)
                        row[key + "_sym_us"] = round(ms * 1e3, 2)
                        row[key + "_sym_busbw"] = round(bus_bandwidth_gbs(nbytes, ms, world)[1], 2)
                        if algo == "auto":
                            row["algo_sym"] = comm.query_algo(nbytes, dt, "sum", registered=True)
                    except Exception as e:  # an algorithm may not apply to a size
                        row[key + "_sym_err"] = str(e)[:80]
                p = plain[:n]
                p.copy_(init[:n] if n <= init.numel() else init.repeat((n + init.numel() - 1) // init.numel())[:n])
                p_out = p if world > 1 else torch.empty_like(p)  # one rank: out of place, so that a kernel runs
                try:
                    ms = _time_loop(lambda: comm.all_reduce(p, "sum", out=p_out, scale=scale, algo=algo), iters, warm, world, reps)
                    row[key + "_us"] = round(ms * 1e3, 2)
                    row[key + "_busbw"] = round(bus_bandwidth_gbs(nbytes, ms, world)[1], 2)
                    if algo == "auto":
                        row["algo"] = comm.query_algo(nbytes, dt, "sum", registered=False)
                except Exception as e:
                    row[key + "_err"] = str(e)[:80]
            if graphs and world > 1 and nbytes <= (1 << 20):
                # Launch-latency-free number: 20 collectives captured in one CUDA graph.
                try:
                    t = sym[dt_name][:n]
                    g = torch.cuda.CUDAGraph()
                    s = torch.cuda.Stream()
                    s.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(s):
                        comm.all_reduce(t, "sum", scale=scale)
                        torch.cuda.synchronize()
                        with torch.cuda.graph(g, stream=s):
                            for _ in range(20):
                                comm.all_reduce(t, "sum", scale=scale)
                    torch.cuda.current_stream().wait_stream(s)
                    ms = _time_loop(lambda: g.replay(), max(3, iters // 10), 2, world) / 20
                    row["ours_graph_us"] = round(ms * 1e3, 2)
                    del g
                except Exception as e:
                    row["ours_graph_err"] = str(e)[:80]
            if with_nccl and world > 1:
                q = plain[:n]
                ms = _time_loop(lambda: dist.all_reduce(q), iters, warm, world, reps)
                row["nccl_us"] = round(ms * 1e3, 2)
                row["nccl_busbw"] = round(bus_bandwidth_gbs(nbytes, ms, world)[1], 2)
                if graphs and nbytes <= (1 << 20):
                    try:
                        g = torch.cuda.CUDAGraph()
                        s = torch.cuda.Stream()
                        s.wait_stream(torch.cuda.current_stream())
                        with torch.cuda.stream(s):
                            dist.all_reduce(q)
                            torch.cuda.synchronize()
                            with torch.cuda.graph(g, stream=s):
                                for _ in range(20):
                                    dist.all_reduce(q)
                        torch.cuda.current_stream().wait_stream(s)
                        ms = _time_loop(lambda: g.replay(), max(3, iters // 10), 2, world) / 20
                        row["nccl_graph_us"] = round(ms * 1e3, 2)
                        del g
                    except Exception as e:
                        row["nccl_graph_err"] = str(e)[:80]
                q.zero_()
                if reg is not None:
                    # NCCL on a buffer from its own registered pool: the partner of "ours, symmetric buffers"
                    qr = reg[:n]
                    qr.zero_()
                    ms = _time_loop(lambda: dist.all_reduce(qr), iters, warm, world, reps)
                    row["nccl_registered_us"] = round(ms * 1e3, 2)
                    row["nccl_registered_busbw"] = round(bus_bandwidth_gbs(nbytes, ms, world)[1], 2)
                elif nccl_registered and isinstance(reg_pool, str):
                    row["nccl_registered_err"] = reg_pool
            rows.append(row)
        del plain
    for t in sym.values():
        comm.free(t)
    return {"note": "device-timed, max over ranks; back-to-back iterations" + (" (quick)" if quick else ""),
            "world": world, "rows": rows}


def main():
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--min-bytes", type=int, default=8 << 10)
    ap.add_argument("--algos", default="auto")
    ap.add_argument("--dtypes", default="fp32,bf16")
    ap.add_argument("--quick", action="store_true")
    ap.add_argument("--no-nccl", action="store_true")
    ap.add_argument("--nccl-registered", action="store_true",
                    help="also time NCCL on a buffer from its own registered pool (ncclMemAlloc through torch.cuda.MemPool)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MINI_NCCL_BOOTSTRAP_PORT" not in os.environ:
        os.environ["MINI_NCCL_BOOTSTRAP_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 17)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import mini_nccl_b200 as mn

    comm = mn.Communicator(world, rank, os.environ["MASTER_ADDR"])
    res = run_sweep(comm, world, rank, max_bytes=args.max_bytes, min_bytes=args.min_bytes, quick=args.quick,
                    dtypes=tuple(args.dtypes.split(",")), algos=tuple(args.algos.split(",")), with_nccl=not args.no_nccl,
                    nccl_registered=args.nccl_registered)
    res["stats"] = comm.stats()
    if rank == 0:
        text = json.dumps(res)
        if args.out:
            with open(args.out, "w") as f:
                f.write(text)
        for r in res["rows"]:
            print(json.dumps(r))
    if world > 1:
        dist.barrier()
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
