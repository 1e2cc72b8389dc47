"""Hera-Core control plane: wire compatibility (checked with raw sockets from Python),
rank assignment, rejection of malformed frames, topology, heartbeat loss and global abort."""
import ctypes as C
import os
import socket
import struct
import subprocess
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
MAGIC = 0x48455241
HDR = struct.Struct("=IBBHI")          # magic, type, version, reserved, payload_len: 12 bytes, host order
REQ = struct.Struct("=64si")           # hostname[64], pid: 68 bytes
RESP = struct.Struct("=ii64s")         # rank, world_size, root_ip[64]: 72 bytes


def recv_exact(s, n):
    buf = b""
    while len(buf) < n:
        chunk = s.recv(n - len(buf))
        if not chunk:
            return buf
        buf += chunk
    return buf


def register_raw(port, hostname=b"pyhost", pid=4242):
    s = socket.create_connection(("127.0.0.1", port), timeout=5)
    s.sendall(HDR.pack(MAGIC, 0x01, 1, 0, REQ.size) + REQ.pack(hostname, pid))
    magic, mtype, ver, rsv, plen = HDR.unpack(recv_exact(s, HDR.size))
    assert (magic, mtype, ver, rsv, plen) == (MAGIC, 0x02, 1, 0, 72)
    rank, world, root = RESP.unpack(recv_exact(s, plen))
    return s, rank, world, root.split(b"\0")[0].decode()


@pytest.fixture
def master(lib, free_port):
    made = []

    def start(world, hb_timeout_ms=0):
        m = lib.mnccl_hera_master_start(world, free_port, hb_timeout_ms)
        assert m
        made.append(m)
        return m, lib.mnccl_hera_master_port(m)

    yield start
    for m in made:
        lib.mnccl_hera_master_stop(m)


def test_wire_sizes():
    assert HDR.size == 12 and REQ.size == 68 and RESP.size == 72


def test_register_wire_format_and_arrival_order(lib, master):
    m, port = master(3)
    conns = []
    for i in range(3):
        s, rank, world, root = register_raw(port, hostname=f"h{i}".encode(), pid=1000 + i)
        conns.append(s)
        assert rank == i, "ranks follow arrival order"
        assert world == 3
        assert root == "127.0.0.1", "root is the first registrant's address as the master sees it"
    time.sleep(0.1)
    assert lib.mnccl_hera_master_registered(m) == 3
    rank, pid, alive = C.c_int(), C.c_int(), C.c_int()
    host, ip = C.create_string_buffer(64), C.create_string_buffer(64)
    assert lib.mnccl_hera_master_worker(m, 1, C.byref(rank), C.byref(pid), host, ip, C.byref(alive)) == 0
    assert (rank.value, pid.value, host.value, ip.value) == (1, 1001, b"h1", b"127.0.0.1")
    # a fourth registrant does not get a rank: the world is full
    s = socket.create_connection(("127.0.0.1", port), timeout=5)
    s.sendall(HDR.pack(MAGIC, 0x01, 1, 0, REQ.size) + REQ.pack(b"late", 1))
    s.settimeout(0.5)
    try:
        assert s.recv(12) == b""
    except (socket.timeout, TimeoutError, ConnectionResetError):
        pass
    for c in conns:
        c.close()


@pytest.mark.parametrize("frame", [
    HDR.pack(0xDEADBEEF, 0x01, 1, 0, REQ.size) + REQ.pack(b"x", 1),      # bad magic
    HDR.pack(MAGIC, 0x01, 2, 0, REQ.size) + REQ.pack(b"x", 1),           # version mismatch
    HDR.pack(MAGIC, 0x01, 1, 0, 8) + b"12345678",                        # short payload for the type
    HDR.pack(MAGIC, 0x01, 1, 0, 0x7FFFFFFF),                             # absurd length
    HDR.pack(MAGIC, 0x77, 1, 0, 0),                                      # unknown type
    HDR.pack(MAGIC, 0x05, 1, 0, 12) + b"\0" * 12,                        # heartbeat before registration
])
def test_malformed_frames_are_rejected(lib, master, frame):
    m, port = master(2)
    s = socket.create_connection(("127.0.0.1", port), timeout=5)
    s.sendall(frame)
    time.sleep(0.3)
    assert lib.mnccl_hera_master_registered(m) == 0
    s.close()
    # the master is still healthy
    s2, rank, world, _ = register_raw(port)
    assert rank == 0 and world == 2
    s2.close()


def test_worker_retries_until_master_appears(lib, free_port):
    import threading

    out = {}

    def late_master():
        time.sleep(0.6)
        out["m"] = lib.mnccl_hera_master_start(1, free_port, 0)

    t = threading.Thread(target=late_master)
    t.start()
    rank, size = C.c_int(-1), C.c_int(-1)
    root = C.create_string_buffer(64)
    w = lib.mnccl_hera_worker_register(b"127.0.0.1", free_port, C.byref(rank), C.byref(size), root)
    t.join()
    assert w and rank.value == 0 and size.value == 1 and root.value == b"127.0.0.1"
    lib.mnccl_hera_worker_free(w)
    lib.mnccl_hera_master_stop(out["m"])


def test_topology_heartbeat_and_global_abort(lib, master):
    m, port = master(3, hb_timeout_ms=0)
    workers = []
    for i in range(3):
        rank, size = C.c_int(), C.c_int()
        root = C.create_string_buffer(64)
        w = lib.mnccl_hera_worker_register(b"127.0.0.1", port, C.byref(rank), C.byref(size), root)
        assert w and rank.value == i
        workers.append(w)
    prev, nxt = C.c_int(), C.c_int()
    ip = C.create_string_buffer(64)
    assert lib.mnccl_hera_worker_topology(workers[2], C.byref(prev), C.byref(nxt), ip) == 0
    assert (prev.value, nxt.value, ip.value) == (1, 0, b"127.0.0.1")
    for i, w in enumerate(workers):
        assert lib.mnccl_hera_worker_start_agent(w, 50, 10 + i) == 0
    time.sleep(0.3)
    assert lib.mnccl_hera_master_abort_sent(m) == 0
    assert lib.mnccl_hera_worker_send_abort(workers[1], 7) == 0      # rank 1 asks for a global abort
    deadline = time.time() + 3
    while time.time() < deadline and not all(lib.mnccl_hera_worker_abort_seen(10 + i) for i in range(3)):
        time.sleep(0.02)
    seen = [lib.mnccl_hera_worker_abort_seen(10 + i) for i in range(3)]
    assert seen == [1000 + 2 * 10 + 7] * 3, seen                      # origin rank 1, reason 7, on every worker
    assert lib.mnccl_hera_master_abort_sent(m) == 1
    for w in workers:
        lib.mnccl_hera_worker_free(w)


def test_lost_keepalive_worker_triggers_abort(lib, master):
    m, port = master(2, hb_timeout_ms=300)
    ws = []
    for i in range(2):
        rank, size = C.c_int(), C.c_int()
        root = C.create_string_buffer(64)
        ws.append(lib.mnccl_hera_worker_register(b"127.0.0.1", port, C.byref(rank), C.byref(size), root))
    assert lib.mnccl_hera_worker_start_agent(ws[0], 50, 20) == 0
    assert lib.mnccl_hera_worker_start_agent(ws[1], 50, 21) == 0
    time.sleep(0.3)
    lib.mnccl_hera_worker_free(ws[1])                                  # rank 1 "dies" (host-side: its socket closes)
    deadline = time.time() + 3
    while time.time() < deadline and not lib.mnccl_hera_worker_abort_seen(20):
        time.sleep(0.02)
    assert lib.mnccl_hera_worker_abort_seen(20) == 1000 + 2 * 10 + 2   # origin rank 1, reason 2 (connection lost)
    lib.mnccl_hera_worker_free(ws[0])


def test_hera_programs(free_port):
    exe = ROOT / "mini_nccl_b200" / "bin" / "hera_test"
    if not exe.exists():
        from mini_nccl_b200 import build

        build.build()
    r = subprocess.run([str(exe), str(free_port)], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0 and "[PASS]" in r.stdout, r.stdout + r.stderr
    # hera_master <world> [port] serves raw clients too
    mexe = ROOT / "mini_nccl_b200" / "bin" / "hera_master"
    p = subprocess.Popen([str(mexe), "1", str(free_port + 1)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
    try:
        for _ in range(50):
            try:
                s, rank, world, root = register_raw(free_port + 1)
                break
            except OSError:
                time.sleep(0.1)
        assert (rank, world) == (0, 1)
        s.close()
    finally:
        p.terminate()
        p.wait(timeout=10)
    assert subprocess.run([str(mexe)], capture_output=True).returncode == 1  # usage
