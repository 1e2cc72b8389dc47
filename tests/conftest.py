import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MINI_NCCL_DEBUG", "WARN")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs at least one CUDA device (run on the GPU box)")
    config.addinivalue_line("markers", "multigpu(n): needs at least n CUDA devices")


def _gpu_count() -> int:
    try:
        import torch

        return torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:
        return 0


def pytest_collection_modifyitems(config, items):
    n = _gpu_count()
    for item in items:
        m = item.get_closest_marker("multigpu")
        if m is not None:
            need = m.args[0] if m.args else 2
            item.add_marker(pytest.mark.gpu)
            if n < need:
                item.add_marker(pytest.mark.skip(reason=f"needs {need} GPUs, have {n}"))
        elif item.get_closest_marker("gpu") is not None and n == 0:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))


@pytest.fixture(scope="session")
def lib():
    import mini_nccl_b200

    return mini_nccl_b200.lib()


_port = [21000 + (os.getpid() % 500) * 16]


@pytest.fixture
def free_port():
    """A TCP port nobody else in this test session uses."""
    import socket

    for _ in range(200):
        _port[0] += 1
        with socket.socket() as s:
            try:
                s.bind(("127.0.0.1", _port[0]))
                return _port[0]
            except OSError:
                continue
    raise RuntimeError("no free port")
