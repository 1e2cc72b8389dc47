"""In-tree native build of libmini_nccl.so and the command-line programs.

Every CUDA translation unit is compiled for sm_100a only
(``-gencode arch=compute_100a,code=sm_100a``); host files with g++.  Objects
are cached under ``build/`` by source mtime, compilation runs in parallel.
The shared library is written to ``mini_nccl_b200/lib/libmini_nccl.so`` and
links the static CUDA runtime, so it loads on machines without a GPU driver
(the network data plane and all host components work there).

The reference builds with CMake and needs libibverbs and libnvToolsExt at
configure time (reference: CMakeLists.txt:21-23); neither is required here:
verbs support is compiled only when <infiniband/verbs.h> exists and NVTX is
header-only.  A CMakeLists.txt at the repository root builds the same targets
for C / C++ users.
"""
from __future__ import annotations

import concurrent.futures as cf
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "csrc"
BUILD = ROOT / "build"
LIBDIR = ROOT / "mini_nccl_b200" / "lib"
BINDIR = ROOT / "mini_nccl_b200" / "bin"

CUDA_HOME = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda"))
NVCC = str(CUDA_HOME / "bin" / "nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]

HOST_SOURCES = [
    "core/log.cc", "core/config.cc",
    "bootstrap/socket.cc", "bootstrap/store.cc", "bootstrap/fdpass.cc", "bootstrap/hera.cc",
    "net/soft_transport.cc", "net/nic_select.cc", "net/ring.cc", "net/factory.cc",
    "mem/cuda_driver.cc", "mem/symmetric.cc",
    "algo/select.cc", "watchdog/watchdog.cc", "ref/oracle.cc", "ref/oracle_api.cc",
    "comm.cc", "api.cc",
]
# Entry points for the test-suite only: linked, with all of the above, into a library of their own
# (libmini_nccl_testhooks.so), so that the product library exports the API and nothing else.
TESTHOOK_SOURCES = ["testing/hooks.cc"]
CUDA_SOURCES = [
    "kernels/k_small.cu", "kernels/k_twoshot.cu", "kernels/k_rsag.cu", "kernels/k_nvls.cu", "kernels/k_pipe.cu", "kernels/k_auto.cu",
    "kernels/launch.cu", "emu/emu_world.cu",
]
# Translation units compiled when present (a source tree may be trimmed to the collectives alone).
OPTIONAL_CUDA = ["kernels/gemm_sm100.cu", "kernels/gemm_fused.cu", "kernels/noalloc.cu", "kernels/elementwise.cu"]
OPTIONAL_HOST = ["net/verbs_transport.cc"]

_HERA_SRCS = ["csrc/bootstrap/hera.cc", "csrc/bootstrap/socket.cc", "csrc/core/log.cc"]
PROGRAMS = {
    # name -> (sources relative to ROOT, links libmini_nccl + CUDA runtime)
    # The Hera programs are self-contained (no CUDA, no shared library), like the
    # reference's header-only control plane.
    "hera_master": (["apps/hera_master.cpp", *_HERA_SRCS], False),
    "hera_test": (["apps/hera_test.cpp", *_HERA_SRCS], False),
    "demo_dual_process": (["apps/demo_dual_process.cpp", "csrc/bootstrap/socket.cc", "csrc/bootstrap/store.cc",
                           "csrc/core/log.cc", "csrc/core/config.cc", "csrc/net/soft_transport.cc", "csrc/net/factory.cc"], False),
    "app": (["apps/app.cpp"], True),
    "perf_test": (["apps/perf_test.cpp"], True),
}


def _have_verbs() -> bool:
    return any(Path(p, "infiniband", "verbs.h").exists() for p in ("/usr/include", "/usr/local/include"))


def _common_includes() -> list[str]:
    return ["-I", str(CSRC), "-I", str(ROOT / "include"), "-I", str(CUDA_HOME / "include")]


def _obj_path(src: Path) -> Path:
    tag = hashlib.sha1(str(src).encode()).hexdigest()[:8]
    return BUILD / f"{src.stem}-{tag}.o"


def _newest_header_mtime() -> float:
    newest = 0.0
    for pat in ("**/*.h", "**/*.cuh"):
        for h in CSRC.glob(pat):
            newest = max(newest, h.stat().st_mtime)
    for h in (ROOT / "include").glob("*.h"):
        newest = max(newest, h.stat().st_mtime)
    return newest


def _compile(src: Path, hdr_mtime: float, verbose: bool, extra: list[str]) -> Path:
    obj = _obj_path(src)
    if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr_mtime):
        return obj
    if src.suffix == ".cu":
        cmd = [NVCC, "-std=c++17", "-O3", *ARCH, "-lineinfo", "-Xcompiler", "-fPIC,-fvisibility=hidden",
               *_common_includes(), *extra, "-c", str(src), "-o", str(obj)]
    else:
        cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-ffp-contract=off", "-Wall", "-Wextra",
               "-pthread", *_common_includes(), *extra, "-c", str(src), "-o", str(obj)]
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {src}\n{r.stdout}\n{r.stderr}")
    if r.stderr.strip() and verbose:
        print(r.stderr, file=sys.stderr)
    return obj


def lib_path() -> Path:
    return LIBDIR / "libmini_nccl.so"


def build(verbose: bool = False, programs: bool = True, jobs: int | None = None) -> Path:
    """Build the shared library (and the programs).  Returns the library path."""
    if not Path(NVCC).exists():
        raise RuntimeError(f"nvcc not found at {NVCC}")
    BUILD.mkdir(exist_ok=True)
    LIBDIR.mkdir(parents=True, exist_ok=True)
    BINDIR.mkdir(parents=True, exist_ok=True)
    extra: list[str] = []
    host = list(HOST_SOURCES)
    cuda = list(CUDA_SOURCES)
    for o in OPTIONAL_CUDA:
        if (CSRC / o).exists():
            cuda.append(o)
    if _have_verbs() and (CSRC / "net/verbs_transport.cc").exists():
        host.append("net/verbs_transport.cc")
        extra.append("-DMNCCL_HAVE_VERBS=1")
    srcs = [CSRC / s for s in host + cuda]
    hdr = _newest_header_mtime()
    jobs = jobs or max(1, (os.cpu_count() or 4))
    with cf.ThreadPoolExecutor(max_workers=jobs) as ex:
        objs = list(ex.map(lambda s: _compile(s, hdr, verbose, extra), srcs))
    lib = lib_path()
    newest_obj = max(o.stat().st_mtime for o in objs)
    if not lib.exists() or lib.stat().st_mtime < newest_obj:
        cmd = [NVCC, "-shared", *ARCH, "-cudart", "static", "-Xlinker", "-Bsymbolic-functions",
               "-o", str(lib), *map(str, objs), "-lpthread", "-lrt", "-ldl"]
        if "-DMNCCL_HAVE_VERBS=1" in extra:
            cmd.append("-libverbs")
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed\n{r.stdout}\n{r.stderr}")
    hooks = LIBDIR / "libmini_nccl_testhooks.so"
    hook_objs = [_compile(CSRC / h, hdr, verbose, extra) for h in TESTHOOK_SOURCES if (CSRC / h).exists()]
    if hook_objs and (not hooks.exists() or hooks.stat().st_mtime < max(newest_obj, max(o.stat().st_mtime for o in hook_objs))):
        cmd = [NVCC, "-shared", *ARCH, "-cudart", "static", "-Xlinker", "-Bsymbolic-functions",
               "-o", str(hooks), *map(str, objs), *map(str, hook_objs), "-lpthread", "-lrt", "-ldl"]
        if "-DMNCCL_HAVE_VERBS=1" in extra:
            cmd.append("-libverbs")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link of the test hooks failed\n{r.stdout}\n{r.stderr}")
    if programs:
        for name, (sources, needs_cuda) in PROGRAMS.items():
            paths = [ROOT / s for s in sources]
            if not all(p.exists() for p in paths):
                continue
            out = BINDIR / name
            newest = max([p.stat().st_mtime for p in paths] + [lib.stat().st_mtime, hdr])
            if out.exists() and out.stat().st_mtime >= newest:
                continue
            cmd = ["g++", "-std=c++17", "-O2", "-mavx2", "-pthread", *_common_includes(), *map(str, paths),
                   "-o", str(out)]
            if needs_cuda:
                cmd += ["-L", str(LIBDIR), "-lmini_nccl", "-Wl,-rpath,$ORIGIN/../lib",
                        "-L", str(CUDA_HOME / "lib64"), "-lcudart_static", "-ldl", "-lrt"]
            if verbose:
                print(" ".join(cmd), flush=True)
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"program build failed: {name}\n{r.stdout}\n{r.stderr}")
    return lib


def build_devcheck_variant(verbose: bool = False, jobs: int | None = None) -> Path:
    """The checked build: the collective kernels compiled with -DMNCCL_DEVICE_CHECKS=1 (every staging
    access is tested against its area and alignment first; a bad one is recorded in the status word and
    skipped, never trapped) and linked with the normal host objects into libmini_nccl_devcheck.so.  The
    stand-in for compute-sanitizer where that tool is not available."""
    lib = build(verbose=verbose, programs=False)
    out = LIBDIR / "libmini_nccl_devcheck.so"
    hdr = _newest_header_mtime()
    checked = ["kernels/k_small.cu", "kernels/k_twoshot.cu", "kernels/k_rsag.cu", "kernels/k_nvls.cu", "kernels/k_pipe.cu", "kernels/k_auto.cu",
               "kernels/launch.cu", "emu/emu_world.cu"]

    def compile_checked(rel: str) -> Path:
        src = CSRC / rel
        obj = BUILD / f"devcheck-{src.stem}.o"
        if obj.exists() and obj.stat().st_mtime >= max(src.stat().st_mtime, hdr):
            return obj
        cmd = [NVCC, "-std=c++17", "-O3", *ARCH, "-lineinfo", "-DMNCCL_DEVICE_CHECKS=1", "-Xcompiler", "-fPIC,-fvisibility=hidden",
               *_common_includes(), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"compile failed: {src}\n{r.stderr}")
        return obj

    with cf.ThreadPoolExecutor(max_workers=jobs or max(1, (os.cpu_count() or 4))) as ex:
        objs = list(ex.map(compile_checked, checked))
    others = [s for s in HOST_SOURCES] + [c for c in CUDA_SOURCES + OPTIONAL_CUDA if c not in checked and (CSRC / c).exists()]
    objs += [_obj_path(CSRC / s) for s in others]
    if not out.exists() or out.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        cmd = [NVCC, "-shared", *ARCH, "-cudart", "static", "-Xlinker", "-Bsymbolic-functions", "-o", str(out),
               *map(str, objs), "-lpthread", "-lrt", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed\n{r.stdout}\n{r.stderr}")
    return out


def build_fake_verbs_variant(verbose: bool = False) -> Path:
    """Test-only variant of the library with the verbs provider compiled against the stand-in
    header and implementation under tests/fake_verbs (no libibverbs needed).  Reuses the objects
    of the normal build; only the transport factory and the provider are compiled again."""
    lib = build(verbose=verbose, programs=False)
    fake = ROOT / "tests" / "fake_verbs"
    out = LIBDIR / "libmini_nccl_fakeverbs.so"
    extra = ["-DMNCCL_HAVE_VERBS=1", "-I", str(fake)]
    special = {CSRC / "net/factory.cc", CSRC / "net/verbs_transport.cc", fake / "fake_verbs.cc"}
    objs = []
    hdr = _newest_header_mtime()
    for s in special:
        o = BUILD / f"fakeverbs-{s.stem}.o"
        if not o.exists() or o.stat().st_mtime < max(s.stat().st_mtime, hdr):
            cmd = ["g++", "-std=c++17", "-O2", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra", "-pthread",
                   *_common_includes(), *extra, "-c", str(s), "-o", str(o)]
            r = subprocess.run(cmd, capture_output=True, text=True)
            if r.returncode != 0:
                raise RuntimeError(f"compile failed: {s}\n{r.stderr}")
        objs.append(o)
    host = [s for s in HOST_SOURCES if s != "net/factory.cc"]
    cuda = list(CUDA_SOURCES) + [o for o in OPTIONAL_CUDA if (CSRC / o).exists()]
    objs += [_obj_path(CSRC / s) for s in host + cuda]
    if not out.exists() or out.stat().st_mtime < max(o.stat().st_mtime for o in objs):
        cmd = [NVCC, "-shared", *ARCH, "-cudart", "static", "-Xlinker", "-Bsymbolic-functions", "-o", str(out),
               *map(str, objs), "-lpthread", "-lrt", "-ldl"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"link failed\n{r.stdout}\n{r.stderr}")
    return out


SELFTEST_SOURCES = ["core/log.cc", "core/config.cc", "bootstrap/socket.cc", "bootstrap/store.cc", "bootstrap/fdpass.cc",
                    "bootstrap/hera.cc", "net/soft_transport.cc", "net/nic_select.cc", "net/ring.cc", "net/factory.cc",
                    "algo/select.cc", "watchdog/watchdog.cc", "ref/oracle.cc", "ref/oracle_api.cc", "testing/hooks.cc",
                    "testing/selftest_main.cc"]


def build_sanitized_selftest(kind: str = "address") -> Path:
    """Host self-test (csrc/testing/selftest_main.cc) compiled with -fsanitize=address,undefined
    (kind="address") or -fsanitize=thread (kind="thread").  No CUDA code is involved."""
    flags = {"address": ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined"], "thread": ["-fsanitize=thread"]}[kind]
    BUILD.mkdir(exist_ok=True)
    out = BUILD / f"host_selftest_{kind}"
    srcs = [CSRC / s for s in SELFTEST_SOURCES]
    newest = max([s.stat().st_mtime for s in srcs] + [_newest_header_mtime()])
    if out.exists() and out.stat().st_mtime >= newest:
        return out
    cmd = ["g++", "-std=c++17", "-O1", "-g", "-fno-omit-frame-pointer", "-ffp-contract=off", "-pthread", "-DMNCCL_HOST_ONLY_SELFTEST=1", *flags,
           *_common_includes(), *map(str, srcs), "-o", str(out), "-lrt", "-ldl"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"sanitized build failed\n{r.stderr[-4000:]}")
    return out


def clean() -> None:
    shutil.rmtree(BUILD, ignore_errors=True)
    for p in (lib_path(),):
        if p.exists():
            p.unlink()


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "clean":
        clean()
    else:
        print(build(verbose="-v" in sys.argv))
