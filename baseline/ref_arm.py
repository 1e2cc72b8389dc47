"""Reference arm of bench.py: times the UNMODIFIED reference library through its own C ABI.

What runs: ``baseline/_ref/libref_mini_nccl.so`` (built by baseline/build_reference.py from a byte
copy of the reference's sources) called exactly the way the reference's own benchmark calls it
(reference: tests/perf_test.cpp:46-153): one process per rank, ``ncclCommInitRank`` with a manual
rank, send / recv buffers from ``cudaHostAlloc`` (pinned host memory), input all 1.0, out-of-place
fp32 sum ``ncclAllReduce`` on a stream, warm-up calls, then K timed calls with a host clock around
the launches plus one final ``cudaStreamSynchronize``, and the check that every element equals the
number of ranks.  Two differences, both on the caller's side: each rank uses its own GPU
(LOCAL_RANK) where the reference's program pins every rank to GPU 0, and the message size, K and
the warm-up count come from bench.py's command line.

This process loads neither this repository's library nor torch: only libcudart, the reference
library and (for the clock record) NVML.  The verbs layer under the reference is the stand-in of
tests/fake_verbs (an RDMA write is a process_vm_writev into the peer process); real RDMA hardware
or Soft-RoCE is unavailable on the machines this runs on, and the output line says so.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import socket
import struct
import sys
import threading
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_LIB = os.path.join(ROOT, "baseline", "_ref", "libref_mini_nccl.so")


def _unavailable(why: str) -> int:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        sys.stdout.flush()
    return 0


class _Gather:
    """Tiny all-gather of one double over TCP through rank 0 (no torch in this process)."""

    def __init__(self, rank, world, addr, port):
        self.rank, self.world = rank, world
        self.socks = []
        if world == 1:
            return
        if rank == 0:
            srv = socket.socket()
            srv.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
            srv.bind((addr, port))
            srv.listen(world)
            srv.settimeout(120)
            for _ in range(world - 1):
                s, _a = srv.accept()
                s.settimeout(600)
                self.socks.append(s)
            srv.close()
        else:
            deadline = time.time() + 120
            while True:
                try:
                    s = socket.create_connection((addr, port), timeout=5)
                    break
                except OSError:
                    if time.time() > deadline:
                        raise
                    time.sleep(0.1)
            s.settimeout(600)
            self.socks.append(s)

    @staticmethod
    def _recv(s, n):
        b = b""
        while len(b) < n:
            c = s.recv(n - len(b))
            if not c:
                raise ConnectionError("peer closed")
            b += c
        return b

    def max(self, v: float) -> float:
        """Maximum over ranks (also a barrier)."""
        if self.world == 1:
            return v
        if self.rank == 0:
            vals = [v] + [struct.unpack("d", self._recv(s, 8))[0] for s in self.socks]
            m = max(vals)
            for s in self.socks:
                s.sendall(struct.pack("d", m))
            return m
        self.socks[0].sendall(struct.pack("d", v))
        return struct.unpack("d", self._recv(self.socks[0], 8))[0]


class _Clocks:
    def __init__(self, dev):
        self.samples, self.sm_max, self._stop, self._t = [], None, threading.Event(), None
        try:
            import pynvml as nv

            nv.nvmlInit()
            self.nv, self.h = nv, nv.nvmlDeviceGetHandleByIndex(dev)
            self.sm_max = int(nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM))
        except Exception:
            self.nv = None

    def _loop(self):
        while not self._stop.is_set():
            try:
                sm = int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                rs = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                self.samples.append((sm, rs))
            except Exception:
                pass
            time.sleep(0.05)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._loop, daemon=True)
            self._t.start()
        return self

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join(timeout=2)
        bits = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
                0x80: "hw_power_brake_slowdown"}
        busy = [s for s in self.samples if not s[1] & 1] or self.samples
        if not busy:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        mask = 0
        for s in busy:
            mask |= s[1]
        sms = sorted(s[0] for s in busy)
        return {"sm_mhz": sms[len(sms) // 2], "sm_max_mhz": self.sm_max, "reasons": [n for b, n in bits.items() if mask & b],
                "samples": len(busy)}


def main(nbytes: int, steps: int, warmup: int) -> int:
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    addr = os.environ.get("MASTER_ADDR", "127.0.0.1")
    port = int(os.environ.get("MASTER_PORT", "29500")) + 31
    if not os.path.exists(REF_LIB):
        return _unavailable("baseline/_ref/libref_mini_nccl.so is missing: the reference tree was not present when "
                            "baseline/build_reference.py ran")
    # The reference overruns its own 1024-deep send queue on large messages (up to
    # WINDOW * SIGNAL_BATCH * 2 requests in flight; reference: src/mini_nccl.cu:119,141-148); the
    # stand-in's queue-depth model is switched off so that it runs to completion anyway.
    os.environ["FAKE_VERBS_SQ_DEPTH_CHECK"] = "0"
    try:
        rt = C.CDLL("libcudart.so.12", mode=C.RTLD_GLOBAL)
    except OSError:
        rt = C.CDLL("/usr/local/cuda/lib64/libcudart.so.12", mode=C.RTLD_GLOBAL)
    ref = C.CDLL(REF_LIB, mode=C.RTLD_LOCAL)
    ref.ncclGetErrorString.restype = C.c_char_p
    ref.ncclCommInitRank.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_char_p]
    ref.ncclAllReduce.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    ref.ncclCommDestroy.argtypes = [C.c_void_p]
    rt.cudaGetErrorString.restype = C.c_char_p

    def cu(code, what):
        if code != 0:
            raise RuntimeError("%s: %s" % (what, rt.cudaGetErrorString(code).decode()))

    ndev = C.c_int(0)
    cu(rt.cudaGetDeviceCount(C.byref(ndev)), "cudaGetDeviceCount")
    cu(rt.cudaSetDevice(local_rank % max(ndev.value, 1)), "cudaSetDevice")
    gather = _Gather(rank, world, addr, port)
    comm = C.c_void_p()
    r = ref.ncclCommInitRank(C.byref(comm), world, rank, b"127.0.0.1")
    ok = gather.max(float(r))
    if ok != 0:
        return _unavailable("reference ncclCommInitRank failed: %s" % ref.ncclGetErrorString(int(r or ok)).decode())
    stream = C.c_void_p()
    cu(rt.cudaStreamCreate(C.byref(stream)), "cudaStreamCreate")
    count = nbytes // 4
    send, recv = C.c_void_p(), C.c_void_p()
    cu(rt.cudaHostAlloc(C.byref(send), C.c_size_t(nbytes), 0), "cudaHostAlloc")
    cu(rt.cudaHostAlloc(C.byref(recv), C.c_size_t(nbytes), 0), "cudaHostAlloc")
    import numpy as np

    a_send = np.ctypeslib.as_array(C.cast(send, C.POINTER(C.c_float)), shape=(count,))
    a_recv = np.ctypeslib.as_array(C.cast(recv, C.POINTER(C.c_float)), shape=(count,))
    a_send[:] = 1.0
    a_recv[:] = 0.0
    NCCL_FLOAT, NCCL_SUM = 7, 0
    failed = 0.0
    why = ""

    def step():
        return ref.ncclAllReduce(send, recv, C.c_size_t(count), NCCL_FLOAT, NCCL_SUM, comm, stream)

    for _ in range(max(warmup, 1)):
        r = step()
        if r != 0:
            failed, why = 1.0, ref.ncclGetErrorString(r).decode()
            break
    rt.cudaStreamSynchronize(stream)
    if gather.max(failed) != 0:
        return _unavailable("reference ncclAllReduce failed during warm-up: %s (bounded by the reference's own "
                            "10 s watchdog; not run again)" % (why or "on another rank"))
    e0, e1 = C.c_void_p(), C.c_void_p()
    cu(rt.cudaEventCreate(C.byref(e0)), "cudaEventCreate")
    cu(rt.cudaEventCreate(C.byref(e1)), "cudaEventCreate")
    clocks = _Clocks(local_rank % max(ndev.value, 1)).start()
    gather.max(0.0)  # barrier
    t0 = time.perf_counter()
    rt.cudaEventRecord(e0, stream)
    for _ in range(steps):
        r = step()
        if r != 0:
            failed, why = 1.0, ref.ncclGetErrorString(r).decode()
            break
    rt.cudaEventRecord(e1, stream)
    rt.cudaStreamSynchronize(stream)
    wall_ms = (time.perf_counter() - t0) * 1e3 / steps
    dev_ms = C.c_float(0)
    rt.cudaEventElapsedTime(C.byref(dev_ms), e0, e1)
    clk = clocks.stop()
    if gather.max(failed) != 0:
        return _unavailable("reference ncclAllReduce failed in the timed loop: %s" % (why or "on another rank"))
    # the reference's own check (reference: tests/perf_test.cpp:102-134): every element == nRanks
    bad = int(np.count_nonzero(np.abs(a_recv - float(world)) > 1e-5))
    bad_all = gather.max(float(bad))
    ms = gather.max(max(wall_ms, dev_ms.value / steps))
    alg = nbytes / (ms * 1e-3) / 1e9
    bus = alg * 2.0 * (world - 1) / world if world > 1 else alg
    if rank == 0:
        line = {
            "metric": "allreduce_busbw_GBps", "value": round(bus, 4), "unit": "GB/s", "n_gpus": world, "steps": steps,
            "warmup": max(warmup, 1), "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "fp32", "data": "synthetic: all 1.0 (the reference benchmark's input)",
            "impl": "reference", "algbw_GBps": round(alg, 4),
            "config": {"model": "AllReduce sum, %d MiB per rank" % (nbytes >> 20), "global_batch": nbytes * world,
                       "seq_len": count, "parallelism": "allreduce x%d" % world,
                       "buffers": "pinned host memory from cudaHostAlloc, as in the reference's perf_test",
                       "timing": "host clock around K blocking calls plus a final stream synchronize (the reference's "
                                 "method); the call is host-synchronous, so this is also the device time; max over ranks",
                       "bus_bandwidth_at_one_rank": "algorithm bandwidth of the degenerate call (factor 2(n-1)/n is 0)",
                       "reference_transport": "stand-in verbs (process_vm_writev, queue-depth model off); real RDMA / "
                                              "Soft-RoCE unavailable on this box",
                       "reference_knobs": "defaults: SLICE_SIZE=131072, WINDOW=64, SIGNAL_BATCH=16"},
            "clocks": clk,
            "e2e": {"value": round(bus, 4), "unit": "GB/s", "ms_per_step": round(ms, 4), "h2d_bytes_per_step": nbytes,
                    "d2h_bytes_per_step": nbytes,
                    "api": "ncclAllReduce on pinned host buffers: the reference's only mode of use; its kernels read the "
                           "input from and write the result to host memory across PCIe every call"},
            "verified": {"elements_wrong": int(bad_all), "rule": "every element == n_ranks within 1e-5"},
            "gpu_launches": 0,
        }
        print(json.dumps(line))
        sys.stdout.flush()
    gather.max(0.0)
    ref.ncclCommDestroy(comm)
    return 0


if __name__ == "__main__":
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--bytes", type=int, default=256 << 20)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    a = ap.parse_args()
    try:
        sys.exit(main(a.bytes, a.steps, a.warmup))
    except Exception as e:  # never a traceback instead of the JSON line
        _unavailable("reference arm stopped: %s" % str(e)[:200])
        sys.exit(0)
