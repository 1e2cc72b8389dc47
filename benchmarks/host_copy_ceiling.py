"""What the host side of the machine can carry: every rank copies a message from pinned host memory to
its GPU and, at the same time on a second stream, a message of the same size back, with plain
``cudaMemcpyAsync`` calls and NO collective.  This is the ceiling for the end-to-end AllReduce on
host-resident buffers (bench.py, key "e2e": per step the input's host-to-device copy and the result's
device-to-host copy are inside the timed region): with N GPUs behind one host the copies share PCIe
switches, the memory controllers and the root complex, so the time per step grows with N although
every GPU has its own link.

  python benchmarks/host_copy_ceiling.py                                # one GPU
  python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/host_copy_ceiling.py

Prints one JSON line: milliseconds per step (maximum over ranks, median of the repeats) and the
aggregate host traffic in GB/s, per chunking of the copies (one copy per direction, or chunks of the
size the library's host pipeline uses).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def measure(nbytes: int, chunk: int, steps: int, repeats: int, world: int) -> float:
    import torch
    import torch.distributed as dist

    from mini_nccl_b200.utils.timing import max_over_ranks

    n = nbytes // 4
    host_in = torch.empty(n, dtype=torch.float32).pin_memory()
    host_out = torch.empty(n, dtype=torch.float32).pin_memory()
    dev_in = torch.empty(n, dtype=torch.float32, device="cuda")
    dev_out = torch.ones(n, dtype=torch.float32, device="cuda")
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    step_elems = n if chunk <= 0 else max(1, chunk // 4)

    def step():
        for off in range(0, n, step_elems):
            end = min(n, off + step_elems)
            with torch.cuda.stream(s_in):
                dev_in[off:end].copy_(host_in[off:end], non_blocking=True)
            with torch.cuda.stream(s_out):
                host_out[off:end].copy_(dev_out[off:end], non_blocking=True)

    seen = []
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    for _ in range(repeats):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        cur = torch.cuda.current_stream()
        e0.record(cur)
        s_in.wait_event(e0)
        s_out.wait_event(e0)
        for _ in range(steps):
            step()
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        e1.record(cur)
        torch.cuda.synchronize()
        seen.append(max_over_ranks(e0.elapsed_time(e1) / steps))
    return sorted(seen)[(len(seen) - 1) // 2]


def main():
    import torch
    import torch.distributed as dist

    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--repeats", type=int, default=5)
    ap.add_argument("--chunks", default="0,8388608,33554432", help="copy chunk sizes in bytes (0 = one copy per direction)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", torch.cuda.current_device()))
    out = {"n_gpus": world, "bytes_each_way_per_rank": args.bytes, "ms_per_step": {}, "aggregate_host_GBps": {}}
    for c in [int(x) for x in args.chunks.split(",")]:
        ms = measure(args.bytes, c, args.steps, args.repeats, world)
        key = "one_copy" if c <= 0 else "%dMiB_chunks" % (c >> 20)
        out["ms_per_step"][key] = round(ms, 4)
        out["aggregate_host_GBps"][key] = round(world * 2 * args.bytes / (ms * 1e-3) / 1e9, 1)
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
