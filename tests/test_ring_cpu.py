"""The network data plane without a GPU: ranks are processes on this machine, the
transport is the soft one-sided provider on loopback, buffers are host memory.
Covers the 2-rank 1 Mi fp32 plumbing configuration (128 KB slices, window 64, signal
batch 16, seeds 1234+rank, AVX2 verifier at 1e-5), odd sizes and rank counts, every
data type and operator, tiny slices (credit and window back-pressure), Hera rank=-1
bootstrap and a host-made transport fault."""
import pytest

from mini_nccl_b200 import _lib
from tests.mp_workers import run_ranks

ALL_DTYPES = list(range(10))


@pytest.mark.parametrize("cma", [0, 1], ids=["sockets", "cross_memory_attach"])
def test_plumbing_config_two_ranks(free_port, cma):
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_SLICE_SIZE": 131072, "MINI_NCCL_WINDOW_SIZE": 64,
           "MINI_NCCL_SIGNAL_BATCH": 16, "MINI_NCCL_SOFT_CMA": cma, "MINI_NCCL_DEBUG": "INFO"}
    cases = [{"dtype": _lib.FLOAT32, "op": _lib.SUM, "count": 1048576, "repeat": 3}]
    res = run_ranks("cpu_ring", 2, {"cases": cases}, env)
    for r in res:
        assert r["cases"] == 1 and r["max_err"] <= 1e-5
        st = r["stats"]
        assert st["plane"] == "soft" and st["algo"]["ring"] == 3
        assert st["ring"]["slice_bytes"] == 131072 and st["ring"]["slots"] == 64
        # 2 MiB chunks -> 16 slices per step, 2 steps per call, 3 calls
        assert st["ring"]["slices_sent"] == 16 * 2 * 3
        # every 16th flag write and each chunk's last one are signalled
        assert st["transport"]["signaled"] == 2 * 2 * 3
        # the user buffer is registered once; later calls hit the cache
        assert st["transport"]["reg_hits"] >= 2
        assert "[Config] Loaded: SLICE_SIZE=131072 B, WINDOW=64, BATCH=16" in r["_stderr"]
        if cma == 0:
            assert st["transport"]["direct_writes"] == 0 and st["transport"]["direct_flags"] == 0
        elif "cross-memory attach to 1 same-host peer" in r["_stderr"]:
            # the kernel allowed it: every payload went straight into the peer's memory, and every flag
            # (one per slice sent, one credit per slice received) was one store into the peer's flag page
            assert st["transport"]["direct_writes"] == st["transport"]["writes"] == 16 * 2 * 3
            assert st["transport"]["direct_flags"] == 2 * 16 * 2 * 3
        else:
            assert st["transport"]["direct_writes"] == 0   # not permitted here: sockets, same results


@pytest.mark.parametrize("n", [2, 3, 4])
def test_odd_sizes_and_small_counts(free_port, n):
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port}
    cases = [{"dtype": _lib.FLOAT32, "op": _lib.SUM, "count": c, "in_place": ip}
             for c in (1, 2, 3, 7, 1000003) for ip in (False, True)]
    res = run_ranks("cpu_ring", n, {"cases": cases}, env)
    assert all(r["cases"] == len(cases) for r in res)


def test_every_dtype_and_op(free_port):
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port}
    cases = [{"dtype": d, "op": o, "count": 4099} for d in ALL_DTYPES for o in range(5)]
    res = run_ranks("cpu_ring", 3, {"cases": cases}, env)
    assert all(r["cases"] == 50 for r in res)


@pytest.mark.parametrize("cma", [0, 1], ids=["sockets", "cross_memory_attach"])
def test_tiny_slices_exercise_credits_and_window(free_port, cma):
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_SLICE_SIZE": 512, "MINI_NCCL_WINDOW_SIZE": 2,
           "MINI_NCCL_SIGNAL_BATCH": 1, "MINI_NCCL_SOFT_CMA": cma}
    cases = [{"dtype": _lib.FLOAT32, "op": _lib.SUM, "count": 200000, "repeat": 2},
             {"dtype": _lib.FLOAT64, "op": _lib.MAX, "count": 50001}]
    res = run_ranks("cpu_ring", 3, {"cases": cases}, env)
    for r in res:
        assert r["stats"]["ring"]["slots"] == 2 and r["stats"]["ring"]["slice_bytes"] == 512
        assert r["stats"]["transport"]["completion_errors"] == 0


def test_hera_auto_bootstrap(free_port, lib):
    # rank = -1: the master hands out ranks in arrival order and the root address.
    hera_port = free_port
    m = lib.mnccl_hera_master_start(3, hera_port, 0)
    assert m
    try:
        env = {"MINI_NCCL_BOOTSTRAP_PORT": hera_port + 101, "MINI_NCCL_HERA_PORT": hera_port}
        cases = [{"dtype": _lib.FLOAT32, "op": _lib.SUM, "count": 65537}]
        res = run_ranks("cpu_ring", 3, {"cases": cases, "hera": True}, env)
        assert sorted(r["rank"] for r in res) == [0, 1, 2]
        assert all(r["size"] == 3 for r in res)
        assert lib.mnccl_hera_master_registered(m) == 3
        assert any("Hera Mode Activated" in r["_stderr"] for r in res)
    finally:
        lib.mnccl_hera_master_stop(m)


def test_dropped_flag_write_fails_bounded(free_port):
    # Rank 0's first data flag is lost on the way (made on the host, in the soft provider).
    # Rank 1 waits for it, the wait runs out after the configured bound, and the call returns
    # an error instead of hanging; rank 0 then fails waiting for rank 1's traffic.
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_WATCHDOG_TIMEOUT_MS": 400, "MINI_NCCL_SOCKET_TIMEOUT_MS": 3000}
    res = run_ranks("cpu_ring_fault", 2, {}, env, per_rank_env={0: {"MINI_NCCL_SOFT_DROP_FLAG_AT": 1}})
    for r in res:
        assert r["rc"] == _lib.INTERNAL_ERROR, r
        assert r["rc2"] == _lib.INTERNAL_ERROR, "the failure is sticky"
        assert r["seconds"] < 5.0, "bounded"
    assert any("Watchdog" in r["_stderr"] and "TIMEOUT" in r["_stderr"] for r in res)


@pytest.mark.parametrize("n", [2, 3, 4])
@pytest.mark.parametrize("threaded", [1, 0])
def test_large_messages_send_from_a_second_thread(free_port, n, threaded):
    """Messages of 4 MB and more: the sends of a call run in a second thread while the caller's thread
    receives and reduces (MINI_NCCL_RING_SENDER_THREAD=0: one thread).  Same results either way, with
    counts the rank count does not divide, few scratch slots (credit stalls) and repeated calls."""
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_RING_SENDER_THREAD": threaded, "MINI_NCCL_WINDOW_SIZE": 4}
    cases = [{"dtype": _lib.FLOAT32, "op": _lib.SUM, "count": (1 << 20) + 7, "in_place": True, "repeat": 2},
             {"dtype": _lib.FLOAT32, "op": _lib.MAX, "count": (3 << 19) + 1},
             {"dtype": _lib.BFLOAT16, "op": _lib.AVG, "count": (1 << 21) + 5},
             {"dtype": _lib.INT32, "op": _lib.SUM, "count": 1 << 20, "in_place": True},
             {"dtype": _lib.FLOAT32, "op": _lib.SUM, "count": 1000}]          # a small one in between: one thread
    res = run_ranks("cpu_ring", n, {"cases": cases}, env, timeout=240)
    for r in res:
        assert r["cases"] == len(cases)
        assert r["stats"]["ring"]["threaded_calls"] == (5 if threaded else 0)
        assert r["stats"]["transport"]["completion_errors"] == 0


def test_dropped_flag_in_a_threaded_call_fails_bounded(free_port):
    """The host-made fault of the test above in a call whose sends run in the second thread: both threads
    of both ranks give up within the bound, the threads are joined, the failure is sticky."""
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_WATCHDOG_TIMEOUT_MS": 400, "MINI_NCCL_SOCKET_TIMEOUT_MS": 3000}
    res = run_ranks("cpu_ring_fault", 2, {"count": 1 << 21}, env, per_rank_env={0: {"MINI_NCCL_SOFT_DROP_FLAG_AT": 9}})
    for r in res:
        assert r["rc"] == _lib.INTERNAL_ERROR, r
        assert r["rc2"] == _lib.INTERNAL_ERROR, "the failure is sticky"
        assert r["seconds"] < 5.0, "bounded"
    assert any("Watchdog" in r["_stderr"] and "TIMEOUT" in r["_stderr"] for r in res)
