#!/usr/bin/env python
"""Headline benchmark: AllReduce bus bandwidth, the reference benchmark's own metric (reference: tests/perf_test.cpp:140-143).

One "step" is one fp32 sum AllReduce of 256 MiB per rank through the library's
public Python API (Communicator.all_reduce on a tensor from Communicator.empty),
timed on the device with CUDA events, maximum over ranks.  The message is larger
than the 126 MB L2, so iterations do not hit in cache.  `value` is the bus
bandwidth algBW * 2(n-1)/n in GB/s; with one GPU that factor is zero, so the
same metric name carries the algorithm bandwidth of the degenerate out-of-place
call (an HBM copy with the scale fused in) and `config` says so.

The K timed steps are repeated R times (each repeat bracketed by a barrier and
a synchronize); the reported value is the MEDIAN repeat, every repeat is listed,
and the per-step spread of the median repeat is given.  After the timed loops
every algorithm of the library is run on seeded random data and compared with
the host oracle ("checked"); a mismatch makes the exit code non-zero.  The "e2e"
number repeats the metric with, per step, the host-to-device copy of the input
from pinned memory and the device-to-host read of the result inside the timed
region, and relates it to the measured ceiling of plain concurrent copies.  A
sweep over message sizes (this library and NCCL side by side) is attached.

`--impl reference` times the unmodified reference library (baseline/ref_arm.py).
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEADLINE_BYTES = 256 << 20
METRIC = "allreduce_busbw_GBps"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--bytes", type=int, default=HEADLINE_BYTES)
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"])
    ap.add_argument("--repeats", type=int, default=7, help="timed regions of --steps steps; the median is reported")
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-check", action="store_true")
    ap.add_argument("--sweep-max-bytes", type=int, default=1 << 30)
    ap.add_argument("--unregistered", action="store_true", help="headline on ordinary torch tensors (staged path)")
    return ap.parse_args()


def reference_arm(args):
    from baseline import ref_arm

    try:
        return ref_arm.main(args.bytes, args.steps, args.warmup)
    except Exception as e:  # the line must come out whatever happens
        if int(os.environ.get("RANK", "0")) == 0:
            print(json.dumps({"impl": "reference", "unavailable": "reference arm stopped: %s" % str(e)[:200]}))
        return 0


def main():
    args = parse()
    if args.impl == "reference":
        return reference_arm(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus and world > 1:
        args.gpus = world
    torch.cuda.set_device(local_rank)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if "MINI_NCCL_BOOTSTRAP_PORT" not in os.environ:
        os.environ["MINI_NCCL_BOOTSTRAP_PORT"] = str(int(os.environ.get("MASTER_PORT", "29500")) + 17)
    os.environ.setdefault("MINI_NCCL_DEBUG", "WARN")
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    import mini_nccl_b200 as mn
    from mini_nccl_b200.utils.timing import ClockSampler, bus_bandwidth_gbs, max_over_ranks, timed_repeats

    comm = mn.Communicator(world, rank, os.environ["MASTER_ADDR"])
    dtype = torch.float32 if args.dtype == "fp32" else torch.bfloat16
    esz = 4 if args.dtype == "fp32" else 2
    count = args.bytes // esz
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    if args.unregistered or world == 1:
        buf = torch.empty(count, dtype=dtype, device="cuda")
    else:
        buf = comm.empty(count, dtype)
    buf.copy_(torch.randn(count, generator=gen, device="cuda", dtype=torch.float32).to(dtype))
    out = torch.empty(count, dtype=dtype, device="cuda") if world == 1 else buf
    stream = torch.cuda.current_stream()
    steps, warmup, repeats = max(args.steps, 1), max(args.warmup, 3), max(args.repeats, 1)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def step():
        # scale keeps the values bounded over many in-place iterations
        comm.all_reduce(buf, "sum", out=out, scale=1.0 / world if world > 1 else 1.0)

    # ---- headline: device-timed, K steps per repeat, max over ranks, median repeat
    # Untimed pre-warm for ~1 s: clocks and NVLink links leave their idle power states (a cold
    # start measured 15 to 25 % below the steady state), then the W warm-up steps proper.
    # Every rank must issue the SAME number of collectives: whether to go on is decided together
    # (each rank's own clock would let one rank run a batch more than another and leave its kernels
    # without partners).
    t_pre = time.perf_counter()
    go_on = torch.ones(1, device="cuda")
    while True:
        for _ in range(10):
            step()
        torch.cuda.synchronize()
        go_on.fill_(1.0 if time.perf_counter() - t_pre < 1.0 else 0.0)
        if world > 1:
            dist.all_reduce(go_on, op=dist.ReduceOp.MIN)
        if go_on.item() == 0.0:
            break
    for _ in range(warmup):
        step()
    # Clocks are sampled DURING the timed repeats by a thread that makes two NVML reads every 50 ms.
    sampler = ClockSampler(torch.cuda.current_device(), period_s=0.05).start()
    timed = timed_repeats(step, steps, repeats, sync_all, stream)
    clocks = sampler.stop()
    # one more repeat with no sampler thread at all, to show that sampling does not move the number
    quiet = timed_repeats(step, steps, 1, sync_all, stream)
    ms = timed["ms_per_step"]
    alg, bus = bus_bandwidth_gbs(args.bytes, ms, world)
    algo_used = comm.query_algo(args.bytes, dtype, "sum", registered=not (args.unregistered or world == 1))

    # ---- end to end: pinned host input -> device -> AllReduce -> host, every step
    host_in = torch.empty(count, dtype=dtype).pin_memory()
    host_in.copy_(buf.cpu())
    host_out = torch.empty(count, dtype=dtype).pin_memory()
    scale = 1.0 / world if world > 1 else 1.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def e2e_step():
        # The call a user of the reference makes: pinned host buffers handed to the collective
        # (its programs allocate their data with cudaHostAlloc).  Inside, the copy engines bring the
        # input to the device and the result back in chunks that overlap the collective.
        comm.all_reduce(host_in, "sum", out=host_out, scale=scale)

    def serial_step():
        # the same work as three explicit, serialised steps
        buf.copy_(host_in, non_blocking=True)
        comm.all_reduce(buf, "sum", out=out, scale=scale)
        host_out.copy_(out, non_blocking=True)

    s_h2d, s_d2h = torch.cuda.Stream(), torch.cuda.Stream()
    scratch = torch.empty(count, dtype=dtype, device="cuda")

    def ceiling_step():
        # no collective at all: the input's host-to-device copy and the result's device-to-host copy
        # at the same time on two streams -- what the host side of this machine can carry
        s_h2d.wait_stream(stream)
        s_d2h.wait_stream(stream)
        with torch.cuda.stream(s_h2d):
            scratch.copy_(host_in, non_blocking=True)
        with torch.cuda.stream(s_d2h):
            host_out.copy_(out, non_blocking=True)
        stream.wait_stream(s_h2d)
        stream.wait_stream(s_d2h)

    def time_e2e(fn):
        for _ in range(3):
            fn()
        n_steps = max(3, min(steps, 20))
        best = []
        for _ in range(3):
            sync_all()
            t0 = time.perf_counter()
            e0.record(stream)
            for _ in range(n_steps):
                fn()
            e1.record(stream)
            torch.cuda.synchronize()
            wall_ms = (time.perf_counter() - t0) * 1e3 / n_steps
            best.append(max_over_ranks(max(e0.elapsed_time(e1) / n_steps, wall_ms)))
        return sorted(best)[1]  # median of three

    e2e_serial_ms = time_e2e(serial_step)
    e2e_ms = time_e2e(e2e_step)
    # the result really is in host memory: compare the two paths' outputs
    e2e_check = bool(torch.allclose(host_out, out.cpu(), rtol=1e-3, atol=1e-3))
    ceiling_ms = time_e2e(ceiling_step)
    e2e_alg, e2e_bus = bus_bandwidth_gbs(args.bytes, e2e_ms, world)
    sync_all()

    # ---- correctness against the host oracle (outside every timed region)
    checked = None
    if not args.no_check:
        from mini_nccl_b200.utils import verify

        # A check that raises (a failed communicator, say) must not cost the run its JSON line: it is
        # reported as a failed check, and the exit code says so.
        try:
            ar = verify.check_allreduce(comm, world, rank)
            gm = verify.check_fused_gemm(comm, world, rank)
            bad = ar["failed"] + gm["failed"]
            bad_any = int(max_over_ranks(float(bad)))
            checked = {"cases": ar["cases"] + gm["cases"], "failed": bad_any, "nvls": ar["nvls"],
                       "fused_gemm_cases": gm["cases"], "failures": (ar["failures"] + gm["failures"])[:8],
                       "notes": gm.get("notes", []),
                       "rule": "P2P algorithms bit-exact against the rank-ordered host oracle; NVLS within tolerance on random "
                               "data and bit-exact on exactly representable data; fused GEMMs bit-exact on integer operands "
                               "(GEMM->reduce-scatter summed by the switch: ties may round to the other bf16 neighbour)"}
            sync_all()
        except Exception as e:  # noqa: BLE001
            checked = {"cases": 0, "failed": 1, "error": ("%s: %s" % (type(e).__name__, e))[:300]}
            try:
                max_over_ranks(1.0)   # the ranks that did not fail are waiting in this reduction
            except Exception:  # noqa: BLE001
                pass

    # ---- sweep (ours vs NCCL), attached for context
    sweep = None
    # (not after a failed check: the ranks agree on "failed" through the reduction above, so they all skip)
    if not args.no_sweep and not (checked and checked["failed"]):
        from benchmarks.sweep import run_sweep

        try:
            sweep = run_sweep(comm, world, rank, max_bytes=args.sweep_max_bytes, quick=True)
            # the headline once more after the sweep: the two loops must agree
            after = timed_repeats(step, steps, 3, sync_all, stream)
            sweep["headline_again_ms_per_step"] = round(after["ms_per_step"], 5)
        except Exception as e:  # noqa: BLE001
            sweep = {"error": ("%s: %s" % (type(e).__name__, e))[:300]}

    stats = comm.stats()
    rc = 0
    if rank == 0:
        line = {
            "metric": METRIC,
            "value": round(bus, 3),
            "unit": "GB/s",
            "n_gpus": world,
            "steps": steps,
            "warmup": warmup,
            "ms_per_step": round(ms, 5),
            "higher_is_better": True,
            "scaling": "weak",
            "vs_baseline": None,
            "dtype": args.dtype,
            "data": "synthetic: normal(0,1) seeded 1234+rank",
            "impl": "ours",
            "algbw_GBps": round(alg, 3),
            "algorithm": algo_used,
            "repeats": {"n": repeats, "reported": "median", "ms_per_step": timed["repeats_ms_per_step"],
                        "step_us_in_median_repeat": timed["step_us"],
                        "without_clock_sampler_ms_per_step": round(quiet["ms_per_step"], 5)},
            "config": {
                "model": "AllReduce sum, %d MiB per rank" % (args.bytes >> 20),
                "global_batch": args.bytes * world,
                "seq_len": count,
                "parallelism": "allreduce x%d" % world,
                "buffers": "ordinary device memory" if (args.unregistered or world == 1) else "symmetric memory (zero-copy)",
                "l2": "message (%d MiB) larger than the 126 MB L2; no flush needed" % (args.bytes >> 20),
                "timing": "CUDA events on the launching stream, max over ranks, median of %d repeats of %d steps" % (repeats, steps),
                "nvls": bool(stats.get("nvls")),
            },
            "clocks": clocks,
            "e2e": {
                "value": round(e2e_bus, 3),
                "unit": "GB/s",
                "ms_per_step": round(e2e_ms, 4),
                "h2d_bytes_per_step": args.bytes,
                "d2h_bytes_per_step": args.bytes,
                "api": "Communicator.all_reduce on pinned host tensors (input and result in host memory)",
                "serialised_copy_collective_copy_ms_per_step": round(e2e_serial_ms, 4),
                "result_matches_device_path": e2e_check,
                "host_copy_ceiling_ms_per_step": round(ceiling_ms, 4),
                "fraction_of_host_copy_ceiling": round(ceiling_ms / e2e_ms, 3) if e2e_ms > 0 else None,
                "ceiling": "the same two copies (256 MiB in, 256 MiB out, pinned memory) at once on two streams on every "
                           "rank, no collective",
            },
            "checked": checked,
            "gpu_launches": steps,
            "gpu_launches_note": "one collective kernel per step in each timed region of %d steps (%d regions)" % (steps, repeats),
            "sweep": sweep,
        }
        if world == 1:
            line["config"]["one_gpu"] = ("bus-bandwidth factor 2(n-1)/n is 0 for one rank: the value is the algorithm bandwidth "
                                         "of the degenerate out-of-place call (HBM copy with the scale fused in)")
        print(json.dumps(line))
        sys.stdout.flush()
    if checked is not None and checked["failed"]:
        rc = 3
    if world > 1 and not (checked and checked["failed"]):
        dist.barrier()
    comm.destroy()
    if world > 1:
        dist.destroy_process_group()
    return rc


if __name__ == "__main__":
    sys.exit(main())
