"""The NVLink data plane with one process per GPU (needs >= 2 GPUs).

`gpu_battery` checks every algorithm (LL, one-shot, two-shot, NVLS when the box
offers multicast, auto) on ordinary and on symmetric buffers against the host
oracle, the fused cast, ReduceScatter / AllGather, pinned host buffers and CUDA
graph capture + replay.  `gpu_stall` is the bounded-failure scenario: a rank stops
launching (a stall made on the host, between steps); the peers' kernels wait, the
watchdog sets the shared abort word after the configured bound, every kernel
returns, and every rank reports an error.  NVLS is off in the stall tests: a rank
that leaves while its memory is bound to a multicast object can fault its peers.
"""
import pytest

from mini_nccl_b200 import _lib
from tests.mp_workers import run_ranks


def _ngpus():
    import torch

    return torch.cuda.device_count()


@pytest.mark.multigpu(2)
def test_battery_two_ranks(free_port):
    res = run_ranks("gpu_battery", 2, {}, {"MINI_NCCL_BOOTSTRAP_PORT": free_port}, timeout=600)
    for r in res:
        assert r["cases"] > 40 and r["plane"] == "nvlink"
        assert r["algo_8k"] == "ll" and r["algo_1m"] == "oneshot" and r["algo_256m"] == "twoshot"
        assert r["stats"]["progress"]["status"] == 0


@pytest.mark.multigpu(2)
def test_battery_ipc_provider_without_nvls(free_port):
    # The fallback provider: cudaMalloc + CUDA IPC handles, no multicast.
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_SYMM": "ipc"}
    res = run_ranks("gpu_battery", 2, {}, env, timeout=600)
    for r in res:
        assert r["provider"] == "ipc" and not r["nvls"]


@pytest.mark.multigpu(4)
def test_battery_all_gpus(free_port):
    n = min(_ngpus(), 8)
    res = run_ranks("gpu_battery", n, {}, {"MINI_NCCL_BOOTSTRAP_PORT": free_port}, timeout=900)
    assert len(res) == n


@pytest.mark.multigpu(2)
def test_hera_bootstrap_and_stall_bounded_failure(free_port, lib):
    # rank = -1 for every process; 1000 AllReduces of 64 KB bf16 in CUDA graphs; the victim
    # stops launching at iteration 500.  Bound: watchdog 1.5 s.
    n = min(_ngpus(), 8)
    hera_port = free_port
    m = lib.mnccl_hera_master_start(n, hera_port, 0)
    assert m
    try:
        env = {"MINI_NCCL_BOOTSTRAP_PORT": hera_port + 211, "MINI_NCCL_HERA_PORT": hera_port,
               "MINI_NCCL_WATCHDOG_TIMEOUT_MS": 1500, "MINI_NCCL_NVLS_ENABLE": 0, "NCCL_NVLS_ENABLE": 0}
        res = run_ranks("gpu_stall", n, {"hera": True, "iters": 1000, "stall_at": 500, "victim": 1}, env, timeout=300)
    finally:
        lib.mnccl_hera_master_stop(m)
    assert sorted(r["rank"] for r in res) == list(range(n))
    for r in res:
        assert r["async"] == _lib.INTERNAL_ERROR, r
        assert r["rc_after"] == _lib.INTERNAL_ERROR, "the communicator stays failed"
        assert r["sync_seconds"] < 30, "every kernel returned within the bound"
        assert not r["stats"]["nvls"]
    tripped = sum(r["stats"]["watchdog"]["trips"] + r["stats"]["watchdog"]["device_failures"] for r in res)
    assert tripped >= 1, "at least one watchdog saw the hang"
    assert any("TIMEOUT DETECTED" in r["_stderr"] or "reported status" in r["_stderr"] for r in res)


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("M", [1024, 256])
@pytest.mark.parametrize("in_switch", [1, 0])
def test_fused_tensor_parallel_kernels(free_port, in_switch, M):
    """Both forms of GEMM -> reduce-scatter: partial tiles summed by the switch (where it can), or pushed
    to their owner and summed there.  M = 1024: 512 rows per rank, CTA pairs; M = 256: 128 rows per rank,
    single-CTA tiles (with their own communication CTAs in the switch form)."""
    n = 2
    res = run_ranks("gpu_tp", n, {"M": M, "N": 1024, "K": 512},
                    {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_RS_SWITCH": in_switch}, timeout=300)
    assert len(res) == n and all(r["worst"] < 3e-2 for r in res)
    if not in_switch:
        assert not any(r["rs_in_switch"] for r in res)


@pytest.mark.multigpu(2)
def test_fused_kernel_stall_fails_the_communicator_within_the_bound(free_port):
    # NVLS off: a rank that leaves while its memory is bound to a multicast object can fault its peers.
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_WATCHDOG_TIMEOUT_MS": 1500, "MINI_NCCL_NVLS_ENABLE": 0,
           "NCCL_NVLS_ENABLE": 0}
    res = run_ranks("gpu_tp_stall", 2, {"victim": 1}, env, timeout=300)
    by_rank = {r["rank"]: r for r in res}
    waiter = by_rank[0]
    assert waiter["waited"] < 20, "the kernel returned within the bound"
    assert waiter["gemm_status"] != 0, "the kernel recorded its failed wait"
    assert waiter["stats"]["watchdog"]["trips"] + waiter["stats"]["watchdog"]["device_failures"] >= 1
    for r in res:
        assert r["async"] == _lib.INTERNAL_ERROR, r
        assert r["raised"] == _lib.INTERNAL_ERROR, "a failed communicator takes no more fused kernels"
        assert not r["stats"]["nvls"]


@pytest.mark.multigpu(8)
def test_fused_tensor_parallel_kernels_llama_shape(free_port):
    # Llama-3-8B block at TP=8: 4096 tokens, hidden 4096, FFN 14336 / 8 = 1792 per rank
    res = run_ranks("gpu_tp", 8, {"M": 4096, "N": 4096, "K": 1792, "iters": 2}, {"MINI_NCCL_BOOTSTRAP_PORT": free_port}, timeout=600)
    assert len(res) == 8


@pytest.mark.multigpu(2)
def test_reference_shaped_programs_on_gpus(free_port):
    # `app` and `perf_test` through the C ABI, one process per GPU; pinned host buffers as in the
    # reference's programs, then device buffers.
    import os
    import subprocess
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    bindir = root / "mini_nccl_b200" / "bin"
    if not (bindir / "app").exists():
        from mini_nccl_b200 import build

        build.build()
    env = dict(os.environ, MINI_NCCL_BOOTSTRAP_PORT=str(free_port))
    ps = [subprocess.Popen([str(bindir / "app"), str(r), "127.0.0.1", "2"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
          for r in range(2)]
    outs = [p.communicate(timeout=180) for p in ps]
    assert all(p.returncode == 0 for p in ps), outs
    assert all("[PASS]" in o[0] and "= 3.0" in o[0] for o in outs)
    for k, dev in enumerate(("0", "1")):
        env2 = dict(env, MINI_NCCL_BOOTSTRAP_PORT=str(free_port + 1 + k), PERF_TEST_MAX_MIB="64", PERF_TEST_DEVICE_BUFFERS=dev)
        ps = [subprocess.Popen([str(bindir / "perf_test"), str(r), "2", "127.0.0.1"], env=env2, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
              for r in range(2)]
        outs = [p.communicate(timeout=300) for p in ps]
        assert all(p.returncode == 0 for p in ps), outs
        assert "BusBW(GB/s)" in outs[0][0] and "67108864" in outs[0][0] and "(FAIL)" not in outs[0][0]
        print(outs[0][0])


@pytest.mark.multigpu(2)
@pytest.mark.parametrize("on", [1, 0])
def test_ordinary_buffers_become_direct_after_first_sight(free_port, on):
    """Lazy direct access: buffers that come back are exported and mapped without a collective call, the
    kernel agrees per call whether it can use them directly; switched off, everything stays staged."""
    res = run_ranks("gpu_auto_map", 2, {"expect_direct": bool(on)},
                    {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_AUTO_MAP": on}, timeout=300)
    assert len(res) == 2 and all(r["cases"] == 8 for r in res)
    if on:
        assert all(r["auto_map"]["direct_calls"] >= 4 for r in res), [r["steps"] for r in res]
    else:
        assert all(r["pipelined_calls"] >= 1 for r in res)
