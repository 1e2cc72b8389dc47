"""Ranks that share ONE GPU: the layout of the reference's benchmark, which pins every rank to GPU 0
(reference: tests/perf_test.cpp:46).  Kernels of different processes on one GPU can never be assumed to
run at the same time, so they must not wait for one another: the library takes its host-synchronised
plane (staging exchanged over CUDA IPC, one reduce kernel per rank between two host barriers).  Needs a
single GPU."""
import os
import subprocess
from pathlib import Path

import pytest

from tests.mp_workers import run_ranks

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [2, 4])
def test_ranks_on_one_gpu_match_the_oracle(free_port, n):
    env = {"MINI_NCCL_BOOTSTRAP_PORT": free_port, "MINI_NCCL_STAGING_BYTES": 16 << 20}   # the big case needs two pieces
    res = run_ranks("gpu_shared", n, {"big": (5 << 20) + 7}, env, timeout=300)
    assert len(res) == n
    for r in res:
        assert r["plane"] == "shared-gpu" and r["cases"] == 21 and r["hostsync"] >= 21
    print("device-buffer AllReduce of 64 MiB, %d ranks on one GPU: %.1f GB/s" % (n, min(r["algbw_GBps"] for r in res)))


def test_perf_test_program_with_every_rank_on_gpu0(free_port):
    """The reference-compatible benchmark program in the reference's own layout: 4 ranks, all on GPU 0,
    pinned host buffers, AVX2 verification; then device buffers."""
    root = Path(__file__).resolve().parent.parent
    exe = root / "mini_nccl_b200" / "bin" / "perf_test"
    if not exe.exists():
        from mini_nccl_b200 import build

        build.build()
    for k, dev in enumerate(("0", "1")):
        env = dict(os.environ, MINI_NCCL_BOOTSTRAP_PORT=str(free_port + k), PERF_TEST_SHARE_GPU="1", PERF_TEST_MAX_MIB="64",
                   PERF_TEST_DEVICE_BUFFERS=dev)
        ps = [subprocess.Popen([str(exe), str(r), "4", "127.0.0.1"], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
              for r in range(4)]
        outs = [p.communicate(timeout=300) for p in ps]
        assert all(p.returncode == 0 for p in ps), outs
        assert "BusBW(GB/s)" in outs[0][0] and "67108864" in outs[0][0] and "(FAIL)" not in outs[0][0]
        print(outs[0][0])
