"""Builds the UNMODIFIED reference library (XuDongGong/Mini-NCCL) for the reference arm of bench.py.

The reference's CMake project needs libibverbs and libnvToolsExt at configure time
(reference: CMakeLists.txt:21-23) and an RDMA device at run time
(reference: src/transport/RDMATransport.h:402-458).  Neither exists on the machines this
repository is measured on, so its two translation units (src/mini_nccl.cu, src/api.cpp) and all
of its headers are copied byte for byte into ``baseline/_ref/src_copy`` and compiled with
nvcc / g++ directly against a stand-in ``<infiniband/verbs.h>`` (tests/fake_verbs: an RDMA write
is a process_vm_writev into the peer process, in post order).  NVTX3 is header-only, so
libnvToolsExt is not needed.  Nothing of this repository's library is linked in.

Result: ``baseline/_ref/libref_mini_nccl.so`` exporting the reference's own C ABI
(ncclCommInitRank / ncclAllReduce / ncclCommDestroy ...), plus ``BUILD_INFO.json`` with the
sha256 of every copied source so the "unmodified" claim can be checked.

  python baseline/build_reference.py [/path/to/reference]
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
OUT = ROOT / "baseline" / "_ref"
FAKE = ROOT / "tests" / "fake_verbs"
CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

COPIED = [
    "include/mini_nccl_api.h", "include/mini_nccl.h", "include/Config.h",
    "src/mini_nccl.cu", "src/api.cpp",
    "src/transport/RDMATransport.h", "src/transport/LockFreeQueue.h", "src/transport/Socket.h",
    "src/hera/hera_msg.h", "src/hera/HeraSocket.h", "src/hera/hera_master.h", "src/hera/hera_worker.h",
]


def lib_path() -> Path:
    return OUT / "libref_mini_nccl.so"


def _sha(p: Path) -> str:
    return hashlib.sha256(p.read_bytes()).hexdigest()


def build(reference: str | os.PathLike = "/root/reference", verbose: bool = False) -> Path | None:
    """Copies and compiles the reference.  Returns the library path, or None when the reference
    tree is not present (then an earlier build under baseline/_ref is used as it is)."""
    ref = Path(reference)
    if not (ref / "src" / "mini_nccl.cu").exists():
        return lib_path() if lib_path().exists() else None
    src = OUT / "src_copy"
    info = {"reference": str(ref), "files": {}}
    for rel in COPIED:
        dst = src / rel
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(ref / rel, dst)
        info["files"][rel] = _sha(dst)
        assert info["files"][rel] == _sha(ref / rel)
    inc = ["-I", str(src / "include"), "-I", str(src / "src"), "-I", str(src / "src" / "transport"),
           "-I", str(src / "src" / "hera"), "-I", str(FAKE), "-I", str(CUDA_HOME / "include")]
    objs = []
    cmds = [
        [NVCC, "-std=c++14", "-O3", *ARCH, "-allow-unsupported-compiler", "-Xcompiler", "-fPIC", *inc,
         "-c", str(src / "src" / "mini_nccl.cu"), "-o", str(OUT / "ref_mini_nccl.o")],
        ["g++", "-std=c++14", "-O3", "-fPIC", *inc, "-c", str(src / "src" / "api.cpp"), "-o", str(OUT / "ref_api.o")],
        ["g++", "-std=c++17", "-O2", "-fPIC", "-I", str(FAKE), "-c", str(FAKE / "fake_verbs.cc"),
         "-o", str(OUT / "ref_fake_verbs.o")],
    ]
    for c in cmds:
        if verbose:
            print(" ".join(c), flush=True)
        r = subprocess.run(c, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError("reference build failed:\n" + " ".join(c) + "\n" + r.stdout + r.stderr)
        objs.append(c[-1])
    link = [NVCC, "-shared", *ARCH, "-cudart", "shared", "-o", str(lib_path()), *objs, "-lpthread", "-ldl", "-lrt"]
    r = subprocess.run(link, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("reference link failed:\n" + r.stdout + r.stderr)
    info["flags"] = "nvcc -std=c++14 -O3 -gencode arch=compute_100a,code=sm_100a (reference: CMakeLists.txt:7-14 uses 'native' and -O3)"
    info["verbs"] = "stand-in: tests/fake_verbs (process_vm_writev); real libibverbs / RDMA device unavailable"
    (OUT / "BUILD_INFO.json").write_text(json.dumps(info, indent=1))
    return lib_path()


if __name__ == "__main__":
    print(build(sys.argv[1] if len(sys.argv) > 1 else "/root/reference", verbose=True))
