"""Host code under sanitizers: the self-test program (queue, pool, cache, watchdog, descriptor
passing, Hera master / workers, a three-rank ring whose ranks are threads) is built with
-fsanitize=address,undefined and with -fsanitize=thread and must report nothing."""
import os
import subprocess

import pytest


@pytest.mark.parametrize("kind", ["address", "thread"])
def test_host_selftest_under_sanitizer(kind, free_port):
    from mini_nccl_b200 import build

    exe = build.build_sanitized_selftest(kind)
    env = dict(os.environ, ASAN_OPTIONS="detect_leaks=1:abort_on_error=0", TSAN_OPTIONS="halt_on_error=0:second_deadlock_stack=1",
               UBSAN_OPTIONS="print_stacktrace=1", MINI_NCCL_DEBUG="NONE")
    r = subprocess.run([str(exe), str(free_port)], capture_output=True, text=True, timeout=600, env=env)
    report = r.stdout + r.stderr
    assert r.returncode == 0, report[-6000:]
    assert "[PASS] host self-test" in r.stdout
    for marker in ("ERROR: AddressSanitizer", "WARNING: ThreadSanitizer", "runtime error:", "ERROR: LeakSanitizer"):
        assert marker not in report, report[-6000:]
