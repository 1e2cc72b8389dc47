"""Device-side timing and clock sampling for the benchmarks.

Rules followed everywhere: warm-up first, CUDA events on the launching stream,
a synchronize on both sides, the maximum over ranks for anything multi-GPU.
Clocks and throttle reasons are only READ (NVML queries); nothing here changes
a GPU setting.
"""
from __future__ import annotations

import threading
import time
from statistics import median


def time_cuda(fn, iters: int, warmup: int = 3, stream=None, pre=None) -> float:
    """Average milliseconds per call of ``fn`` over ``iters`` back-to-back calls."""
    import torch

    stream = stream or torch.cuda.current_stream()
    for _ in range(warmup):
        fn()
    if pre is not None:
        pre()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record(stream)
    for _ in range(iters):
        fn()
    stop.record(stream)
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / max(iters, 1)


def timed_repeats(step, steps: int, repeats: int, sync_all, stream=None) -> dict:
    """The benchmark's timed region, `repeats` times over: a barrier and a synchronize, one CUDA event
    before every step and one after the last, `steps` back-to-back calls of ``step``, a synchronize.
    Every repeat's milliseconds per step is the maximum over ranks; the reported figure is the MEDIAN
    repeat, so that neither a one-off stall of a shared machine nor a lucky loop decides the number.
    The per-step durations (this rank's events) of the median repeat tell a slow outlier from a
    uniform slowdown."""
    import torch

    stream = stream or torch.cuda.current_stream()
    per_repeat, per_step = [], []
    for _ in range(repeats):
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(steps + 1)]
        sync_all()
        ev[0].record(stream)
        for i in range(steps):
            step()
            ev[i + 1].record(stream)
        torch.cuda.synchronize()
        per_repeat.append(max_over_ranks(ev[0].elapsed_time(ev[steps]) / steps))
        per_step.append([ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(steps)])
    order = sorted(range(repeats), key=lambda i: per_repeat[i])
    mid = order[(repeats - 1) // 2]
    us = sorted(per_step[mid])
    return {
        "ms_per_step": per_repeat[mid],
        "repeats_ms_per_step": [round(x, 5) for x in per_repeat],
        "step_us": {"min": round(us[0], 1), "median": round(us[len(us) // 2], 1), "max": round(us[-1], 1)},
    }


def max_over_ranks(value: float) -> float:
    """Maximum of a host scalar over all ranks of the default torch.distributed group."""
    import torch
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return value
    dev = "cuda" if dist.get_backend() == "nccl" else "cpu"
    t = torch.tensor([value], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def bus_bandwidth_gbs(nbytes: int, ms: float, nranks: int) -> tuple[float, float]:
    """(algorithm bandwidth, bus bandwidth) in GB/s with the reference benchmark's formulas
    (reference: tests/perf_test.cpp:140-143): alg = bytes / time, bus = alg * 2(n-1)/n."""
    alg = nbytes / (ms * 1e-3) / 1e9 if ms > 0 else 0.0
    bus = alg * 2.0 * (nranks - 1) / nranks if nranks > 1 else alg
    return alg, bus


_REASON_BITS = {
    0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
    0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown", 0x80: "hw_power_brake_slowdown",
    0x100: "display_clock_setting",
}


class ClockSampler:
    """Samples SM clock, power and clock-event reasons of one GPU in a background thread."""

    def __init__(self, device_index: int, period_s: float = 0.02):
        self.device_index = device_index
        self.period_s = period_s
        self.samples: list[tuple[int, float, int]] = []
        self.sm_max = 0
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        self._handle = None

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._nvml = None
            return self
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def _loop(self):
        nv = self._nvml
        while not self._stop.is_set():
            try:
                sm = int(nv.nvmlDeviceGetClockInfo(self._handle, nv.NVML_CLOCK_SM))
                try:
                    pw = nv.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
                except Exception:
                    pw = 0.0
                try:
                    rs = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
                except Exception:
                    try:
                        rs = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
                    except Exception:
                        rs = 0
                self.samples.append((sm, pw, rs))
            except Exception:
                pass
            time.sleep(self.period_s)

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max or None, "reasons": [], "samples": 0}
        # "under load": ignore samples flagged idle when busy ones exist
        busy = [s for s in self.samples if not (s[2] & 0x1)] or self.samples
        mask = 0
        for s in busy:
            mask |= s[2]
        reasons = [name for bit, name in _REASON_BITS.items() if mask & bit and name != "gpu_idle"]
        return {
            "sm_mhz": int(median(s[0] for s in busy)),
            "sm_max_mhz": self.sm_max,
            "power_w_max": round(max(s[1] for s in busy), 1),
            "reasons": reasons,
            "samples": len(busy),
        }
