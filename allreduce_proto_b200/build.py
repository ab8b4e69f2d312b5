"""In-tree build of the native library, the C++ tools and the tests.

Everything is compiled with explicit ``g++`` / ``nvcc`` command lines (CUDA
objects for ``sm_100a`` only) into

* ``allreduce_proto_b200/_lib/libibcomm_cuda.so`` — host transport, CPU
  schedules, device arena, kernels and the C API the Python package loads
* ``allreduce_proto_b200/_lib/libibcomm.so`` — host-only variant
* ``build/bin/`` — ``ibcomm_run``, ``allreduce_tester``, ``allreduce``,
  ``allreduce_cuda``, ``sendrecv``, ``unittest``, ``bench_sweep``

The same targets are described for CMake users in ``CMakeLists.txt``; this
script exists so that ``python -m allreduce_proto_b200.build`` works on a
machine that has nothing but the CUDA toolkit and Python.  Objects are rebuilt
when a source or any header is newer than the object.
"""
from __future__ import annotations

import concurrent.futures
import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
LIB_DIR = ROOT / "allreduce_proto_b200" / "_lib"
BUILD_DIR = ROOT / "build"
BIN_DIR = BUILD_DIR / "bin"
OBJ_DIR = BUILD_DIR / "obj"

HOST_SOURCES = [
    "src/host/error.cpp",
    "src/host/env.cpp",
    "src/host/partition.cpp",
    "src/host/shm_transport.cpp",
    "src/host/trace.cpp",
    "src/host/communicator.cpp",
    "src/host/bootstrap.cpp",
    "src/host/schedule.cpp",
    "src/host/tuner.cpp",
    "src/host/tunables.cpp",
    "src/host/c_api.cpp",
]
CUDA_SOURCES = [
    "src/cuda/driver_api.cpp",
    "src/cuda/fd_channel.cpp",
    "src/cuda/arena.cpp",
    "src/cuda/engine.cpp",
    "src/cuda/device_context.cpp",
    "src/cuda/emu_world.cpp",
    "src/cuda/exec_kernel.cu",
    "src/cuda/nvls_kernel.cu",
    "src/cuda/oneshot_kernel.cu",
    "src/cuda/rsag_kernel.cu",
    "src/cuda/hybrid_kernel.cu",
    "src/cuda/staged_kernel.cu",
    "src/cuda/copy_kernel.cu",
    "src/cuda/p2p_sendrecv.cu",
    "src/cuda/no_alloc.cu",
]
# (binary name, source, needs_cuda)
PROGRAMS = [
    ("ibcomm_run", "apps/ibcomm_run.cpp", False),
    ("allreduce_tester", "apps/allreduce_tester.cpp", True),
    ("bench_sweep", "apps/bench_sweep.cpp", True),
    ("allreduce", "examples/allreduce.cpp", False),
    ("allreduce_cuda", "examples/allreduce.cpp", True),
    ("sendrecv", "tests/cpp/sendrecv_test.cpp", False),
    ("unittest", "tests/cpp/unittest.cpp", False),
    ("schedule_sim", "tests/cpp/schedule_sim.cpp", False),
    ("twoshot_sim", "tests/cpp/twoshot_sim.cpp", False),
    ("threads_test", "tests/cpp/threads_test.cpp", False),
    ("threads_test_cuda", "tests/cpp/threads_test.cpp", True),
]

CXXFLAGS = ["-std=c++17", "-O2", "-g", "-fPIC", "-Wall", "-Wextra", "-pthread", f"-I{ROOT / 'include'}"]
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCCFLAGS = ["-std=c++17", "-O3", "-lineinfo", "-Xcompiler", "-fPIC,-Wall,-pthread", f"-I{ROOT / 'include'}", f"-I{ROOT / 'src' / 'cuda'}",
             "-DUSE_CUDA", "--expt-relaxed-constexpr", "-Xptxas", "-v"] + NVCC_ARCH


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not Path(exe).exists():
        raise RuntimeError("nvcc not found")
    return exe


def _headers_mtime() -> float:
    newest = 0.0
    for pattern in ("include/**/*.h", "src/**/*.h", "src/**/*.cuh"):
        for p in ROOT.glob(pattern):
            newest = max(newest, p.stat().st_mtime)
    return newest


def _stale(out: Path, deps_mtime: float, *srcs: Path) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(s.stat().st_mtime > t for s in srcs) or deps_mtime > t


def _run(cmd, log: Path | None = None) -> None:
    proc = subprocess.run([str(c) for c in cmd], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if log is not None:
        log.write_text(proc.stdout)
    if proc.returncode != 0:
        sys.stderr.write(" ".join(str(c) for c in cmd) + "\n" + proc.stdout)
        raise RuntimeError(f"build step failed: {cmd[0]} {cmd[-1]}")


def _compile(src: str, variant: str, hdr_mtime: float) -> Path:
    """variant: 'host' (g++, no CUDA), 'cuda' (nvcc or g++ with -DUSE_CUDA)."""
    s = ROOT / src
    obj = OBJ_DIR / variant / (src.replace("/", "_") + ".o")
    obj.parent.mkdir(parents=True, exist_ok=True)
    if not _stale(obj, hdr_mtime, s):
        return obj
    if variant == "host":
        _run(["g++", *CXXFLAGS, "-c", s, "-o", obj])
    elif s.suffix == ".cu":
        _run([_nvcc(), *NVCCFLAGS, "-c", s, "-o", obj], log=obj.with_suffix(".ptxas.log"))
    else:
        cuda_inc = Path(_nvcc()).resolve().parent.parent / "include"
        _run(["g++", *CXXFLAGS, "-DUSE_CUDA", f"-I{cuda_inc}", f"-I{ROOT / 'src' / 'cuda'}", "-c", s, "-o", obj])
    return obj


def build(verbose: bool = False, jobs: int | None = None, host_only: bool = False) -> dict:
    """Builds every target that is out of date.  Returns the output paths.

    ``host_only`` skips everything that needs nvcc (the host library, the
    launcher and the host tests are still built).
    """
    for d in (LIB_DIR, BIN_DIR, OBJ_DIR):
        d.mkdir(parents=True, exist_ok=True)
    hdr = _headers_mtime()
    jobs = jobs or min(8, os.cpu_count() or 4)

    host_srcs = [s for s in HOST_SOURCES if (ROOT / s).exists()]
    cuda_srcs = [] if host_only else [s for s in CUDA_SOURCES if (ROOT / s).exists()]
    programs = [p for p in PROGRAMS if (ROOT / p[1]).exists() and not (host_only and p[2])]

    tasks = []
    for s in host_srcs:
        tasks.append((s, "host"))
        if not host_only:
            tasks.append((s, "cuda"))
    for s in cuda_srcs:
        tasks.append((s, "cuda"))
    for _, s, needs_cuda in programs:
        tasks.append((s, "cuda" if needs_cuda else "host"))
    tasks = list(dict.fromkeys(tasks))

    objs: dict = {}
    with concurrent.futures.ThreadPoolExecutor(max_workers=jobs) as pool:
        futs = {pool.submit(_compile, s, v, hdr): (s, v) for s, v in tasks}
        for f in concurrent.futures.as_completed(futs):
            objs[futs[f]] = f.result()
            if verbose:
                print("compiled", *futs[f])

    out = {}
    # host-only library
    lib_host = LIB_DIR / "libibcomm.so"
    host_objs = [objs[(s, "host")] for s in host_srcs]
    if _stale(lib_host, 0, *host_objs):
        _run(["g++", "-shared", "-o", lib_host, *host_objs, "-pthread", "-lrt"])
    out["libibcomm"] = lib_host
    # library with the device paths; cudart is linked statically so the file
    # loads on machines without a driver (CUDA calls then report "no device").
    lib_cuda = LIB_DIR / "libibcomm_cuda.so"
    cuda_objs = [] if host_only else [objs[(s, "cuda")] for s in host_srcs + cuda_srcs]
    if cuda_srcs and _stale(lib_cuda, 0, *cuda_objs):
        _run([_nvcc(), *NVCC_ARCH, "-shared", "-o", lib_cuda, *cuda_objs, "-Xcompiler", "-pthread", "-lrt", "-ldl",
              "-cudart", "static"])
    out["libibcomm_cuda"] = lib_cuda if cuda_srcs else None

    for name, s, needs_cuda in programs:
        exe = BIN_DIR / name
        variant = "cuda" if needs_cuda else "host"
        if needs_cuda and not cuda_srcs:
            continue
        o = objs[(s, variant)]
        lib = lib_cuda if needs_cuda else lib_host
        if _stale(exe, 0, o, lib):
            rpath = f"-Wl,-rpath,{LIB_DIR}"
            if needs_cuda:
                _run([_nvcc(), *NVCC_ARCH, "-o", exe, o, f"-L{LIB_DIR}", "-libcomm_cuda", "-Xlinker",
                      f"-rpath={LIB_DIR}", "-Xlinker", "-rpath=$ORIGIN/../../allreduce_proto_b200/_lib",
                      "-Xcompiler", "-pthread", "-lrt", "-ldl", "-cudart", "static"])
            else:
                _run(["g++", "-o", exe, o, f"-L{LIB_DIR}", "-libcomm", rpath,
                      "-Wl,-rpath,$ORIGIN/../../allreduce_proto_b200/_lib", "-pthread", "-lrt"])
        out[name] = exe
    return out


def ptxas_report() -> str:
    """Concatenated ``-Xptxas -v`` output of every CUDA object (registers, spills, shared memory)."""
    parts = []
    for log in sorted((OBJ_DIR / "cuda").glob("*.ptxas.log")):
        parts.append(f"== {log.name}\n{log.read_text()}")
    return "\n".join(parts)


if __name__ == "__main__":
    res = build(verbose="-v" in sys.argv, host_only="--host-only" in sys.argv)
    for k, v in res.items():
        print(f"{k}: {v}")
