"""Forced-algorithm x launch-tuning sweep, the measurement behind the selection table in
csrc/algo/select.cc.  For every message size each applicable algorithm is timed (device time,
max over ranks) on symmetric and on ordinary buffers, with several grid caps and NVLS unroll
factors; NCCL is timed eagerly and inside a CUDA graph for reference.

With ``--table FILE`` the measured crossovers are written as a tuning table that the library loads at
start-up when MINI_NCCL_TUNING_FILE names it (lines ``<nranks> <KNOB> <value>``; rows of other rank
counts already in the file are kept), so the choice of algorithm follows THIS machine's measured bus
bandwidth; without a table the constants compiled into csrc/algo/select.cc apply.

  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/tune.py --out tune8.json --table tuning.txt
  MINI_NCCL_TUNING_FILE=tuning.txt python ...
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from benchmarks.sweep import _time_loop  # noqa: E402


def _best_time(row: dict, where: str, algo: str):
    """Fastest measured time (us) of `algo` on `where` buffers in a row, over its launch variants."""
    vals = [v for k, v in row.items() if isinstance(v, (int, float)) and not k.endswith("_graph")
            and (k == f"{where}_{algo}" or k.startswith(f"{where}_{algo}_b"))]
    return min(vals) if vals else None


def crossovers(rows: list[dict], where: str = "sym") -> dict:
    """Selection knobs from a sweep: LL up to the largest size where it is the fastest algorithm, one-shot
    up to the largest size where it beats both two-phase kernels, NVLS from the smallest size where it
    beats the peer-to-peer two-shot kernel.  Sizes without a measurement of an algorithm do not vote.
    Pure function of the rows (tested without a GPU)."""
    knobs = {}
    ll_max = oneshot_max = 0
    nvls_min = None
    for row in sorted(rows, key=lambda r: r["bytes"]):
        t = {a: _best_time(row, where, a) for a in ("ll", "oneshot", "twoshot", "nvls")}
        have = {a: v for a, v in t.items() if v is not None}
        if not have:
            continue
        best = min(have, key=have.get)
        if best == "ll":
            ll_max = row["bytes"]
        two_phase = [v for a, v in have.items() if a in ("twoshot", "nvls")]
        if "oneshot" in have and (best in ("ll", "oneshot") or not two_phase or have["oneshot"] <= min(two_phase)):
            oneshot_max = max(oneshot_max, row["bytes"])
        if "nvls" in have and "twoshot" in have and have["nvls"] < have["twoshot"] and nvls_min is None:
            nvls_min = row["bytes"]
    if ll_max:
        knobs["LL_MAX_BYTES"] = ll_max
    if oneshot_max:
        knobs["ONESHOT_MAX_BYTES"] = max(oneshot_max, ll_max)
    if nvls_min is not None:
        knobs["NVLS_MIN_BYTES"] = max(nvls_min, knobs.get("ONESHOT_MAX_BYTES", 0) + 1)
    return knobs


def write_table(path: str, world: int, knobs: dict, note: str = "") -> None:
    """Writes / updates the rows of `world` ranks in a tuning table, keeping the other rank counts' rows."""
    keep = []
    if os.path.exists(path):
        for line in open(path):
            body = line.split("#", 1)[0].split()
            if len(body) == 3 and body[0] == str(world):
                continue
            if line.strip() and not line.startswith("# written by benchmarks/tune.py"):
                keep.append(line.rstrip("\n"))
    with open(path, "w") as f:
        f.write("# written by benchmarks/tune.py: <nranks> <KNOB> <value>; loaded through MINI_NCCL_TUNING_FILE\n")
        for line in keep:
            f.write(line + "\n")
        for k, v in sorted(knobs.items()):
            f.write(f"{world} {k} {int(v)}" + (f"   # {note}" if note else "") + "\n")


def graph_time(fn, world, inner=20, reps=5):
    import torch

    g = torch.cuda.CUDAGraph()
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=s):
            for _ in range(inner):
                fn()
    torch.cuda.current_stream().wait_stream(s)
    ms = _time_loop(lambda: g.replay(), reps, 2, world) / inner
    del g
    return ms


def main():
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--sizes", default="8192,65536,262144,1048576,4194304,16777216,67108864,268435456,1073741824")
    ap.add_argument("--dtype", default="fp32")
    ap.add_argument("--blocks", default="16,24,32,64,96")
    ap.add_argument("--plain", action="store_true", help="also time ordinary (staged) buffers")
    ap.add_argument("--table", default="", help="write the measured crossovers as a tuning table (MINI_NCCL_TUNING_FILE)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MINI_NCCL_BOOTSTRAP_PORT" not in os.environ:
        os.environ["MINI_NCCL_BOOTSTRAP_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 17)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    import mini_nccl_b200 as mn
    from mini_nccl_b200.utils.timing import bus_bandwidth_gbs

    comm = mn.Communicator(world, rank, os.environ["MASTER_ADDR"])
    nvls = bool(comm.stats()["nvls"])
    dt = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    esz = 4 if args.dtype == "fp32" else 2
    sizes = [int(x) for x in args.sizes.split(",")]
    blocks = [int(x) for x in args.blocks.split(",")]
    cap = max(sizes)
    sym = comm.empty(cap // esz, dt)
    plain = torch.empty(cap // esz, dtype=dt, device="cuda")
    sym.normal_()
    plain.normal_()
    rows = []
    scale = 1.0 / world
    for nbytes in sizes:
        n = nbytes // esz
        iters = 100 if nbytes <= (1 << 20) else (30 if nbytes <= (64 << 20) else 8)
        row = {"bytes": nbytes, "dtype": args.dtype, "world": world}
        bufs = [("sym", sym[:n])] + ([("plain", plain[:n])] if args.plain else [])
        for where, t in bufs:
            cands = []
            if nbytes <= 64 * 1024:
                cands.append(("ll", 0, 0))
            if nbytes <= (4 << 20 if world <= 2 else (2 << 20 if world <= 4 else 1 << 20)):
                cands.append(("oneshot", 0, 0))
            if nbytes >= 65536:
                for b in blocks:
                    cands.append(("twoshot", b, 0))
                    if nvls:
                        cands.append(("nvls", b, 4))
                        cands.append(("nvls", b, 8))
            for algo, b, u in cands:
                comm.set_tuning(b, u)
                key = f"{where}_{algo}" + (f"_b{b}" if b else "") + (f"_u{u}" if u else "")
                try:
                    ms = _time_loop(lambda: comm.all_reduce(t, "sum", scale=scale, algo=algo), iters, 3, world)
                    row[key] = round(ms * 1e3, 2)
                    if nbytes <= (1 << 20) and b in (0, blocks[0]) and u in (0, 4):
                        row[key + "_graph"] = round(graph_time(lambda: comm.all_reduce(t, "sum", scale=scale, algo=algo), world) * 1e3, 2)
                except Exception as e:
                    row[key + "_err"] = str(e)[:60]
            comm.set_tuning(0, 0)
        q = plain[:n]
        ms = _time_loop(lambda: dist.all_reduce(q), iters, 3, world)
        row["nccl"] = round(ms * 1e3, 2)
        if nbytes <= (1 << 20):
            row["nccl_graph"] = round(graph_time(lambda: dist.all_reduce(q), world) * 1e3, 2)
        q.normal_()
        best = min((v, k) for k, v in row.items() if isinstance(v, float) and k.startswith("sym_") and not k.endswith("_graph"))
        row["best_sym"] = best[1]
        row["best_sym_busbw"] = round(bus_bandwidth_gbs(nbytes, best[0] / 1e3, world)[1], 1)
        row["nccl_busbw"] = round(bus_bandwidth_gbs(nbytes, row["nccl"] / 1e3, world)[1], 1)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and args.out:
        with open(args.out, "w") as f:
            json.dump({"world": world, "nvls": nvls, "rows": rows}, f)
    if rank == 0 and args.table:
        knobs = crossovers(rows)
        write_table(args.table, world, knobs, note=f"{args.dtype}, symmetric buffers")
        print("tuning table:", json.dumps(knobs), flush=True)
    dist.barrier()
    comm.free(sym)
    comm.destroy()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
