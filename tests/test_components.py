"""Host components one by one: config knobs, SPSC queue, request pool, registration cache,
NIC choice, NUMA parsing, descriptor passing, watchdog logic, the launch planner."""
import ctypes as C
import json

import pytest

from mini_nccl_b200 import _lib


def cfg(lib, env):
    out = C.create_string_buffer(2048)
    rc = lib.mnccl_test_config(env.encode(), out, 2048)
    return rc, (json.loads(out.value.decode()) if rc == 0 else None)


def test_config_defaults_and_banner(lib):
    rc, c = cfg(lib, "")
    assert rc == 0
    assert c["slice_size"] == 131072 and c["window_size"] == 64 and c["signal_batch"] == 16
    assert c["watchdog_timeout_ms"] == 10000 and c["bootstrap_port"] == 8888 and c["hera_port"] == 9999
    assert c["banner"] == "Loaded: SLICE_SIZE=131072 B, WINDOW=64, BATCH=16"


def test_config_clamps(lib):
    rc, c = cfg(lib, "MINI_NCCL_SLICE_SIZE=0;MINI_NCCL_WINDOW_SIZE=-3;MINI_NCCL_SIGNAL_BATCH=0")
    assert rc == 0
    assert c["slice_size"] == 1024   # 0 -> 1024
    assert c["window_size"] == 1     # <= 0 -> 1
    assert c["signal_batch"] == 1    # 0 would be a modulo by zero in the slice loop


def test_config_values_and_suffixes(lib):
    rc, c = cfg(lib, "MINI_NCCL_SLICE_SIZE=64K;MINI_NCCL_WINDOW_SIZE=8;MINI_NCCL_SIGNAL_BATCH=4;MINI_NCCL_NET_DEVICE=mlx5_1;"
                     "MINI_NCCL_WATCHDOG_TIMEOUT_MS=250;MINI_NCCL_ALGO=nvls;MINI_NCCL_NVLS_ENABLE=0")
    assert rc == 0
    assert c["slice_size"] == 65536 and c["window_size"] == 8 and c["signal_batch"] == 4
    assert c["net_device"] == "mlx5_1" and c["watchdog_timeout_ms"] == 250 and c["algo"] == "nvls" and c["nvls_enable"] is False


def test_config_pipeline_knobs(lib):
    rc, c = cfg(lib, "")
    assert rc == 0
    assert c["pipeline_min_bytes"] == 48 << 20 and c["host_pipeline_min_bytes"] == 4 << 20 and c["host_chunk_bytes"] == 8 << 20
    rc, c = cfg(lib, "MINI_NCCL_HOST_PIPELINE_MIN_BYTES=0;MINI_NCCL_HOST_CHUNK_BYTES=1K;MINI_NCCL_PIPELINE_MIN_BYTES=1M")
    assert rc == 0
    assert c["host_pipeline_min_bytes"] == 0          # 0 switches the host pipeline off
    assert c["host_chunk_bytes"] == 64 << 10          # clamped: tiny chunks would be all launch overhead
    assert c["pipeline_min_bytes"] == 1 << 20


@pytest.mark.parametrize("bad", ["MINI_NCCL_SLICE_SIZE=abc", "MINI_NCCL_WINDOW_SIZE=1.5x", "MINI_NCCL_NVLS_ENABLE=maybe",
                                 "MINI_NCCL_BOOTSTRAP_PORT=70000", "MINI_NCCL_SLICE_SIZE=-5"])
def test_config_malformed_is_invalid_argument(lib, bad):
    rc, _ = cfg(lib, bad)
    assert rc == 100 + _lib.INVALID_ARGUMENT


def test_spsc_queue(lib):
    assert lib.mnccl_test_spsc(1, 1000) == 0
    assert lib.mnccl_test_spsc(7, 200000) == 0
    assert lib.mnccl_test_spsc(4096, 500000) == 0


def test_request_pool(lib):
    assert lib.mnccl_test_request_pool(4096) == 0
    assert lib.mnccl_test_request_pool(3) == 0


def test_registration_cache(lib):
    assert lib.mnccl_test_reg_cache() == 0


def test_nic_selection_policy(lib):
    idx = C.c_int(-1)
    assert lib.mnccl_test_select_nic(b"mlx5_0,rxe0,mlx5_1", b"", C.byref(idx)) == 0 and idx.value == 1   # rxe0 first
    assert lib.mnccl_test_select_nic(b"eth_rdma,mlx5_0,mlx5_1", b"", C.byref(idx)) == 0 and idx.value == 1  # then mlx5
    assert lib.mnccl_test_select_nic(b"hfi1_0,bnxt_re0", b"", C.byref(idx)) == 0 and idx.value == 0        # else first
    assert lib.mnccl_test_select_nic(b"mlx5_0,rxe0,mlx5_1", b"mlx5_1", C.byref(idx)) == 0 and idx.value == 2  # override
    assert lib.mnccl_test_select_nic(b"mlx5_0,rxe0", b"nope0", C.byref(idx)) == 100 + _lib.SYSTEM_ERROR     # no match: error
    assert lib.mnccl_test_select_nic(b"", b"", C.byref(idx)) == 100 + _lib.SYSTEM_ERROR                     # no devices


def test_cpu_list_parser(lib):
    out = (C.c_int * 64)()
    n = lib.mnccl_test_parse_cpu_list(b"0-3,8,10-11\n", out, 64)
    assert list(out[:n]) == [0, 1, 2, 3, 8, 10, 11]
    assert lib.mnccl_test_parse_cpu_list(b"", out, 64) == 0
    n = lib.mnccl_test_parse_cpu_list(b"5", out, 64)
    assert list(out[:n]) == [5]
    n = lib.mnccl_test_parse_cpu_list(b"x,2-1,7", out, 64)
    assert list(out[:n]) == [7]


def test_numa_lookup_on_fake_sysfs(lib, tmp_path):
    dev = tmp_path / "class" / "infiniband" / "mlx5_0" / "device"
    dev.mkdir(parents=True)
    (dev / "numa_node").write_text("1\n")
    node = tmp_path / "devices" / "system" / "node" / "node1"
    node.mkdir(parents=True)
    (node / "cpulist").write_text("16-31,48-63\n")
    nd, ncpu = C.c_int(), C.c_int()
    lib.mnccl_test_numa(str(tmp_path).encode(), b"mlx5_0", C.byref(nd), C.byref(ncpu))
    assert nd.value == 1 and ncpu.value == 32
    lib.mnccl_test_numa(str(tmp_path).encode(), b"absent0", C.byref(nd), C.byref(ncpu))
    assert nd.value == -1 and ncpu.value == 0
    (dev / "numa_node").write_text("-1\n")
    lib.mnccl_test_numa(str(tmp_path).encode(), b"mlx5_0", C.byref(nd), C.byref(ncpu))
    assert nd.value == -1 and ncpu.value == 0


def test_descriptor_passing(lib):
    import os

    assert lib.mnccl_test_fdpass(f"t{os.getpid()}".encode()) == 0


def test_watchdog_logic(lib):
    assert lib.mnccl_test_watchdog(0, 100) == 0   # finishes in time: no abort
    assert lib.mnccl_test_watchdog(1, 100) == 1   # stuck past the bound: abort word set, one trip
    assert lib.mnccl_test_watchdog(2, 100) == 1   # a kernel reported a failed wait: abort at once


def plan(lib, n, count, dtype=_lib.FLOAT32, op=_lib.SUM, mode=0, in_sym=0, out_sym=0, nvls=0, forced=0, stage=0, wire=None, out=None):
    algo, nb, cin, cout = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    se, cv = C.c_uint64(), C.c_uint64()
    rc = lib.mnccl_test_plan(n, mode, count, dtype, dtype if wire is None else wire, dtype if out is None else out, op, in_sym,
                             out_sym, nvls, forced, stage, C.byref(algo), C.byref(nb), C.byref(se), C.byref(cv), C.byref(cin), C.byref(cout))
    if rc:
        return None
    return dict(algo=_lib.ALGO_NAMES[algo.value], nblocks=nb.value, shard=se.value, chunk=cv.value, copy_in=cin.value, copy_out=cout.value)


def test_planner_direct_two_shot_for_ordinary_buffers_on_four_gpus(lib):
    """Ordinary device buffers with lazy direct access on (bit 1 of in_sym): four GPUs take the peer-to-peer
    two-shot kernel from 4 MB to below 192 MB, where it measured ahead of the staged switch kernel and of
    the pipelined kernel; other rank counts, sizes and ineligible buffers keep their choice.  The choice
    never depends on what has been mapped so far."""
    mb = 1 << 18  # fp32 elements per MB
    assert plan(lib, 4, 16 * mb, nvls=1, in_sym=2)["algo"] == "twoshot"
    assert plan(lib, 4, 128 * mb, nvls=1, in_sym=2)["algo"] == "twoshot"
    assert plan(lib, 4, 4 * mb, nvls=1, in_sym=2)["algo"] == "twoshot"
    assert plan(lib, 4, 3 * mb, nvls=1, in_sym=2)["algo"] == "nvls"
    assert plan(lib, 4, 2 * mb, nvls=1, in_sym=2)["algo"] == "oneshot"
    assert plan(lib, 4, 256 * mb, nvls=1, in_sym=2)["algo"] == "pipe"
    assert plan(lib, 4, 16 * mb, nvls=1, in_sym=0)["algo"] == "nvls"
    assert plan(lib, 8, 16 * mb, nvls=1, in_sym=2)["algo"] == "nvls"
    assert plan(lib, 2, 16 * mb, nvls=1, in_sym=2)["algo"] == "twoshot"    # two ranks: two-shot anyway
    p = plan(lib, 4, 16 * mb, nvls=1, in_sym=2)
    assert p["copy_in"] == 1 and p["copy_out"] == 1, "planned as the staged kernel; the kernel itself goes direct"


def test_tuning_table_loader(lib):
    """MINI_NCCL_TUNING_FILE: lines '<nranks> <KNOB> <value>'; rows for other rank counts are skipped,
    nranks 0 matches all, comments and blank lines are ignored, bad rows are reported and skipped."""
    import json

    text = """# measured on some machine
8 LL_MAX_BYTES 32768
8 ONESHOT_MAX_BYTES 262144   # crossover to the two-phase kernels
4 ONESHOT_MAX_BYTES 1048576
0 PIPE_MIN_BYTES 16777216

8 NO_SUCH_KNOB 1
8 MAX_BLOCKS 100000
garbage here
"""
    buf = C.create_string_buffer(2048)
    assert lib.mnccl_test_tuning_text(text.encode(), 8, buf, len(buf)) == 0
    got = json.loads(buf.value.decode())
    assert got["applied"] == 3 and got["ll_max_bytes"] == 32768 and got["oneshot_max_bytes"] == 262144
    assert got["pipe_min_bytes"] == 16777216 and got["max_blocks"] == 0
    assert "NO_SUCH_KNOB" in got["errors"] and "MAX_BLOCKS" in got["errors"] and "line 9" in got["errors"]
    assert lib.mnccl_test_tuning_text(text.encode(), 4, buf, len(buf)) == 0
    got = json.loads(buf.value.decode())
    assert got["applied"] == 2 and got["oneshot_max_bytes"] == 1048576 and got["ll_max_bytes"] == 0


def test_tune_script_derives_a_table_the_library_loads(lib, tmp_path):
    """benchmarks/tune.py: crossovers from a (here synthetic) sweep, written as a table, read back by the
    library's loader; rows of another rank count survive an update."""
    import json

    from benchmarks.tune import crossovers, write_table

    rows = [
        {"bytes": 8192, "sym_ll": 9.0, "sym_oneshot": 12.0},
        {"bytes": 65536, "sym_ll": 11.0, "sym_oneshot": 12.5, "sym_twoshot_b32": 20.0, "sym_nvls_b32_u4": 19.0},
        {"bytes": 262144, "sym_oneshot": 14.0, "sym_twoshot_b32": 19.0, "sym_nvls_b32_u4": 16.5, "sym_nvls_b16_u4": 15.0},
        {"bytes": 1048576, "sym_oneshot": 28.0, "sym_twoshot_b32": 24.0, "sym_nvls_b32_u4": 21.0, "sym_oneshot_graph": 1.0},
        {"bytes": 4194304, "sym_twoshot_b96": 40.0, "sym_nvls_b32_u4": 30.0},
    ]
    knobs = crossovers(rows)
    assert knobs == {"LL_MAX_BYTES": 65536, "ONESHOT_MAX_BYTES": 262144, "NVLS_MIN_BYTES": 262145}
    path = tmp_path / "tuning.txt"
    path.write_text("4 ONESHOT_MAX_BYTES 524288\n")
    write_table(str(path), 8, knobs, note="test")
    write_table(str(path), 8, knobs, note="again")            # an update replaces the rows of 8 ranks only
    text = path.read_text()
    assert text.count("8 LL_MAX_BYTES") == 1 and "4 ONESHOT_MAX_BYTES 524288" in text
    buf = C.create_string_buffer(2048)
    assert lib.mnccl_test_tuning_text(text.encode(), 8, buf, len(buf)) == 0
    got = json.loads(buf.value.decode())
    assert got["applied"] == 3 and got["ll_max_bytes"] == 65536 and got["oneshot_max_bytes"] == 262144 and got["nvls_min_bytes"] == 262145
    assert got["errors"] == ""
    assert lib.mnccl_test_tuning_text(text.encode(), 4, buf, len(buf)) == 0
    assert json.loads(buf.value.decode())["oneshot_max_bytes"] == 524288


def test_planner_picks_by_size(lib):
    assert plan(lib, 8, 2048)["algo"] == "ll"                      # 8 KB
    assert plan(lib, 8, 16384)["algo"] == "ll"                     # 64 KB
    assert plan(lib, 8, 40000)["algo"] == "oneshot"                # 160 KB
    assert plan(lib, 8, 1 << 20)["algo"] == "twoshot"              # 4 MB, no multicast
    assert plan(lib, 8, 1 << 18)["algo"] == "oneshot"              # 1 MB on ordinary buffers: no staging copies
    assert plan(lib, 8, 1 << 18, in_sym=1, out_sym=1)["algo"] == "twoshot"
    assert plan(lib, 8, 1 << 20, nvls=1)["algo"] == "nvls"
    assert plan(lib, 8, 1 << 20, nvls=1, op=_lib.MAX)["algo"] == "twoshot"      # the switch only adds
    assert plan(lib, 8, 1 << 20, nvls=1, dtype=_lib.INT32)["algo"] == "twoshot"
    assert plan(lib, 1, 12345)["algo"] == "local"
    assert plan(lib, 8, 1 << 26, forced=_lib.ALGO_LL)["algo"] == "twoshot"      # forced but impossible: degrade


def test_planner_geometry(lib):
    p = plan(lib, 8, 1000003)
    assert p["shard"] % 4 == 0 and p["shard"] * 8 >= 1000003 and (p["shard"] - 4) * 8 < 1000003 + 32
    assert p["copy_in"] == 1 and p["copy_out"] == 1
    z = plan(lib, 8, 1 << 24, in_sym=1, out_sym=1, nvls=1)
    assert z["algo"] == "nvls" and z["copy_in"] == 0 and z["copy_out"] == 0 and z["chunk"] * 4 == z["shard"]
    s = plan(lib, 4, 1 << 26, stage=1 << 20, forced=_lib.ALGO_TWOSHOT)   # 256 MB through 1 MB of staging: many passes
    assert s["chunk"] == (1 << 20) // (4 * 16)
    assert 1 <= s["nblocks"] <= 512
    assert plan(lib, 4, 1000, dtype=_lib.FLOAT32, wire=_lib.INT32) is None   # no such cast
    rs = plan(lib, 4, 1001, mode=1)
    assert rs["algo"] == "twoshot" and rs["shard"] == 1001 and rs["copy_out"] == 0
    ag = plan(lib, 4, 1001, mode=2)
    assert ag["algo"] == "twoshot" and ag["copy_in"] == 0 and ag["copy_out"] == 1


def test_planner_pipelined_kernel_for_large_ordinary_buffers(lib):
    """Ordinary device buffers of 24 MB and more take the pipelined kernel; its chunk is N shards of
    whole vectors and fits one of the 16 ring slots of either staging area."""
    p = plan(lib, 8, 1 << 26, nvls=1)                    # 256 MB fp32, ordinary buffers
    assert p["algo"] == "pipe" and p["copy_in"] == 1 and p["copy_out"] == 1
    assert p["shard"] % 4 == 0 and p["shard"] * 8 * 4 <= (256 << 20) // 16 and 3 <= p["nblocks"] <= 140
    assert plan(lib, 8, 1 << 26, nvls=1, in_sym=1, out_sym=1)["algo"] == "nvls"     # symmetric buffers stay zero-copy
    assert plan(lib, 8, (8 << 20) // 4, nvls=1)["algo"] != "pipe"                    # below the threshold
    assert plan(lib, 2, 1 << 26)["algo"] == "twoshot"     # two ranks keep the stream pipeline around the two-phase kernel
    q = plan(lib, 2, 1 << 26, forced=7)                  # ... unless the pipelined kernel is asked for (peer-to-peer reduction)
    assert q["algo"] == "pipe" and q["shard"] % 4 == 0
    assert plan(lib, 8, 1 << 26, nvls=1, op=_lib.MAX)["algo"] == "twoshot"          # the switch only adds
    m = plan(lib, 8, 1 << 25, nvls=1, wire=_lib.BFLOAT16, out=_lib.FLOAT32)          # fp32 out of a bf16 wire: slot bound by the output
    assert m["algo"] == "pipe" and m["shard"] % 8 == 0 and m["shard"] * 8 * 4 <= (256 << 20) // 16
    t = plan(lib, 4, 1 << 26, nvls=1, stage=1 << 20)     # tiny staging: 16 KB slots
    assert t["algo"] == "pipe" and t["shard"] * 4 * 4 <= (1 << 20) // 64
    assert plan(lib, 8, 1 << 26, mode=1)["algo"] == "twoshot"                        # only AllReduce is pipelined


def test_gemm_split_k_plan_of_the_last_wave(lib):
    """Host arithmetic of the CTA-pair kernel's split-K: only a last wave that leaves at least half of the
    pairs idle is cut, and only where the measured cost model says the cut pays; every slice has at least
    4 k-blocks, all slices fit one wave, none is empty."""
    if not hasattr(lib, "mncclGemmSplitPlan"):
        pytest.skip("library built without the GEMM translation unit")
    f, s, k = C.c_int(), C.c_int(), C.c_int()
    plan_of = lambda M, N, K, pairs=74: (lib.mncclGemmSplitPlan(M, N, K, pairs, C.byref(f), C.byref(s), C.byref(k)), f.value, s.value, k.value)
    ok, first, slices, per = plan_of(4096, 3584, 4096)           # 224 tiles on 74 pairs: 3 waves + 2 tiles
    assert ok == 1 and first == 222 and slices == 8 and per == 8
    assert plan_of(8192, 8192, 8192)[0] == 0                      # 1024 tiles: the last wave holds 62 of 74
    assert plan_of(4096, 4096, 1792)[0] == 0                      # 3 waves + 34 tiles: two slices would save less than the cut costs
    assert plan_of(4096, 4096, 512)[0] == 0
    assert plan_of(4096, 9216, 1792)[0] == 0                      # 576 tiles = 7 waves + 58: more than half of the pairs busy
    assert plan_of(2048, 2048, 4096)[0] == 0                      # 64 tiles: a single wave
    ok, first, slices, per = plan_of(4096, 3584, 256)             # 4 k-blocks: too short to cut
    assert ok == 0
    assert plan_of(4096, 4864, 1024, 74)[0] == 0                  # 16 k-blocks: the tile is shorter than the cut's cost
    ok, first, slices, per = plan_of(4096, 4864, 4096, 74)        # 16 x 19 = 304 tiles = 4 waves + 8; 64 k-blocks
    assert ok == 1 and first == 296 and slices == 8 and per == 8 and slices * 8 <= 74


def test_gemm_host_plan_picks_tiles_and_cta_pairs():
    """Host-side choice of the GEMM kernel (no GPU needed): CTA pairs for products whose 256 x 256
    tiles fill the SM pairs, narrower single-CTA tiles for small products, and the pinned modes."""
    import mini_nccl_b200 as mn
    from mini_nccl_b200.ops.gemm import gemm_plan, set_pair_mode

    if not hasattr(mn.lib(), "mncclGemmPlan"):
        pytest.skip("library built without the GEMM translation unit")
    try:
        set_pair_mode(-1)
        assert gemm_plan(8192, 8192)[1] is True
        assert gemm_plan(4096, 3584)[1] is True          # 224 pair tiles on 74 pairs
        assert gemm_plan(2048, 2048)[1] is True          # 64 pair tiles: most pairs busy
        assert gemm_plan(1024, 1024) == (128, False)     # 16 pair tiles would leave 58 pairs idle
        assert gemm_plan(128, 4096)[1] is False          # fewer than 256 rows: no pair tile
        assert gemm_plan(4096, 128)[1] is False          # fewer than 256 columns
        assert gemm_plan(4096, 4096, ctas=1)[1] is False
        # the tile width is never one the epilogue cannot take
        for m, n in ((4096, 3584), (512, 7168), (300, 1000)):
            assert gemm_plan(m, n, narrow=False)[0] in (256, 192)
            assert gemm_plan(m, n, narrow=True)[0] in (256, 224, 192, 128)
        set_pair_mode(0)
        assert gemm_plan(8192, 8192)[1] is False
        set_pair_mode(1)
        assert gemm_plan(1024, 1024)[1] is True
        assert gemm_plan(128, 4096)[1] is False          # pinned on, but the shape has no pair tile
    finally:
        set_pair_mode(-1)


def test_swiglu_entry_validates_arguments_before_touching_the_gpu(lib):
    if not hasattr(lib, "mncclSwiGluBf16"):
        pytest.skip("library built without csrc/kernels/elementwise.cu")
    assert lib.mncclSwiGluBf16(None, None, 4, 8, 0, 0, None) == -1      # null pointers
    assert lib.mncclSwiGluBf16(16, 32, 0, 8, 0, 0, None) == -1          # empty
    assert lib.mncclSwiGluBf16(16, 32, 4, 6, 0, 0, None) == -2          # F no multiple of 8
    assert lib.mncclSwiGluBf16(8, 32, 4, 8, 0, 0, None) == -2           # input not 16-byte aligned
    assert lib.mncclSwiGluBf16(16, 32, 4, 8, 8, 0, None) == -2          # input row stride shorter than 2F
    assert lib.mncclSwiGluBf16(16, 32, 4, 8, 0, 4, None) == -2          # output row stride no multiple of 8


def _chunks(lib, count, elem_bytes, uniform, cap, taper):
    out = (C.c_size_t * 256)()
    lib.mnccl_test_pipeline_chunks.restype = C.c_int
    lib.mnccl_test_pipeline_chunks.argtypes = [C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.POINTER(C.c_size_t), C.c_int]
    n = lib.mnccl_test_pipeline_chunks(count, elem_bytes, uniform, cap, taper, out, 256)
    assert 0 <= n <= 256, n
    return [out[i] for i in range(n)]


def test_pipeline_chunk_schedule(lib):
    import random

    MB = 1 << 20
    cap = 128 * MB // 4                       # elements of fp32 that fit one half of the staging
    # the regular schedule: equal chunks, the last one takes the rest
    assert _chunks(lib, 64 * MB // 4 + 12345, 4, 32 * MB // 4, cap, 0) == [8 * MB, 8 * MB, 12345]
    assert _chunks(lib, 0, 4, 32 * MB // 4, cap, 0) == []
    # tapering leaves messages below 128 MB alone
    assert _chunks(lib, 64 * MB // 4, 4, 32 * MB // 4, cap, 1) == [8 * MB, 8 * MB]
    # 256 MiB of fp32: 32 MB edges, two equal large chunks between them
    assert _chunks(lib, 256 * MB // 4, 4, 64 * MB // 4, cap, 1) == [8 * MB, 24 * MB, 24 * MB, 8 * MB]
    # 1 GiB: the large chunks fill a staging half or nearly so
    c = _chunks(lib, 1024 * MB // 4, 4, cap, cap, 1)
    assert c[0] == c[-1] == 8 * MB and len(c) == 10 and max(c) <= cap
    # invariants on arbitrary sizes and types
    rng = random.Random(5)
    for _ in range(300):
        esz = rng.choice([1, 2, 4, 8])
        count = rng.randrange(1, (3 << 30) // esz)
        cap_e = (128 * MB // esz) & ~4095
        uni = min(max((count // 4) & ~4095, (32 * MB // esz) & ~4095), cap_e)
        for taper in (0, 1):
            c = _chunks(lib, count, esz, uni, cap_e, taper)
            assert sum(c) == count and all(x > 0 for x in c)
            assert all(x % 4096 == 0 for x in c[:-1]), "every chunk but the last keeps vector alignment of the next"
            assert max(c) <= cap_e + 4095
            if taper and count * esz >= 128 * MB and len(c) >= 3:
                assert c[0] * esz <= 32 * MB and c[-1] * esz <= 32 * MB + 4096 * esz


def _tile_walk(lib, M, N, bn, group_m, rotate, pair, n_workers):
    f = lib.mncclGemmTileOrder
    f.restype = C.c_int
    f.argtypes = [C.c_int] * 8 + [C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int]
    walks = []
    for w in range(n_workers):
        tm, tn = (C.c_int * 8192)(), (C.c_int * 8192)()
        n = f(M, N, bn, group_m, rotate, pair, n_workers, w, tm, tn, 8192)
        assert 0 <= n <= 8192
        walks.append([(tm[i], tn[i]) for i in range(n)])
    return walks


@pytest.mark.parametrize("pair", [0, 1])
@pytest.mark.parametrize("nranks,rank", [(1, 0), (2, 1), (8, 2), (8, 7)])
def test_gemm_tile_walk_covers_every_tile_once_in_owner_order(lib, pair, nranks, rank):
    """The tile order of the fused kernels, computed by the kernels' own index arithmetic on the host:
    every 128-row tile exactly once, work spread evenly, GEMM -> reduce-scatter visits the owners
    starting with the next rank and its own rows last, all-gather -> GEMM starts with the local rows."""
    if not hasattr(lib, "mncclGemmTileOrder"):
        pytest.skip("library built without the GEMM translation unit")
    M, N, bn = 4096, 3584 if pair else 4096, 256
    tiles_m, tiles_n = M // 128, (N + bn - 1) // bn
    local = tiles_m // nranks
    n_workers = 56 if pair else 132
    for name, rotate in (("reduce-scatter", ((rank + 1) % nranks) * local), ("all-gather", rank * local)):
        walks = _tile_walk(lib, M, N, bn, local, rotate, pair, n_workers)
        flat = [t for w in walks for t in w]
        assert sorted(flat) == sorted((m, n) for m in range(tiles_m) for n in range(tiles_n)), name
        sizes = [len(w) for w in walks]
        assert max(sizes) - min(sizes) <= (2 if pair else 1), name
        # global order = round-robin over the workers; the owner of a tile is tm // local
        step = 2 if pair else 1
        order = []
        for k in range(0, max(sizes), step):
            for w in walks:
                order.extend(w[k:k + step])
        owners = [tm // local for tm, _ in order]
        seen = []
        for o in owners:
            if not seen or seen[-1] != o:
                seen.append(o)
        first = (rank + 1) % nranks if name == "reduce-scatter" else rank
        assert seen == [(first + i) % nranks for i in range(nranks)], (name, seen)


@pytest.mark.parametrize("cma", [0, 1], ids=["sockets", "cross_memory_attach"])
def test_soft_provider_rejects_bad_key_and_range(lib, free_port, cma):
    lib.mnccl_test_soft_reject.restype = C.c_int
    rc = lib.mnccl_test_soft_reject(int(free_port), cma)
    if rc == -1:
        pytest.skip("cross-memory attach is not permitted on this machine")
    assert rc == 0, f"check {rc} failed"


def test_switch_tie_rule_accepts_only_true_ties():
    """The oracle check of the in-switch GEMM -> reduce-scatter: the other bf16 neighbour is accepted exactly
    where the exact sum lies halfway between two bf16 values, nowhere else."""
    import numpy as np

    from mini_nccl_b200.utils import oracle as O
    from mini_nccl_b200.utils.verify import switch_ties

    exact = np.array([257.0, 258.0, 259.0, 513.0, 514.0, 100.0, -257.0], dtype=np.float32)
    want = O.f32_to_bf16_bits(exact)                       # nearest-even: 256, 258, 260, 512, 512, 100, -256
    assert list(O.bf16_bits_to_f32(want)) == [256.0, 258.0, 260.0, 512.0, 512.0, 100.0, -256.0]
    other = O.f32_to_bf16_bits(np.array([258.0, 258.0, 258.0, 516.0, 516.0, 100.0, -258.0], dtype=np.float32))
    tie = switch_ties(other, want, exact)
    # 257, 259 and -257 are ties between their neighbours; 513 is not (512 is nearer than 516); 514 is a tie
    assert list(tie) == [True, False, True, False, True, False, True]
    wrong = want.copy()
    wrong[5] = O.f32_to_bf16_bits(np.array([100.5], dtype=np.float32))[0]
    assert not switch_ties(wrong, want, exact).any(), "an ordinary mismatch is never excused"


def test_nccl_registered_buffer_degrades_without_a_process_group():
    """benchmarks/sweep.py --nccl-registered: without NCCL (no GPU, no process group) the helper reports why
    instead of raising, so a sweep simply has no such column."""
    import os
    import sys

    import torch

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    from benchmarks.sweep import nccl_registered_buffer

    t, why = nccl_registered_buffer(1024, torch.float32)
    if t is None:
        assert isinstance(why, str) and why
