"""In-tree native build: compiles every CUDA source for sm_100a and the host runtime with g++.

Two shared libraries are produced under ``llmq_b200/lib``:

* ``libllmq_b200_kernels.so`` - all device kernels and their C launchers (``csrc/*.cu``)
* ``libllmq_b200_rt.so``      - host-side runtime: token-file data loader, safetensors writer,
  bump/stack arena bookkeeping, pinned staging helpers (``csrc/rt/*.cpp``)

The build is incremental (object files are rebuilt only when a source or header is newer) and
needs no GPU: nvcc cross-compiles.  Run ``python -m llmq_b200.build`` or call :func:`build`.
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG = Path(__file__).resolve().parent
CSRC = PKG / "csrc"
LIBDIR = PKG / "lib"
OBJDIR = PKG.parent / "build" / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "--expt-relaxed-constexpr", "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-Wall", "-pthread"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if cand and (os.path.isabs(cand) and os.path.exists(cand) or not os.path.isabs(cand)):
            return cand
    return "nvcc"


def _newest_header_mtime(dirs) -> float:
    m = 0.0
    for d in dirs:
        for ext in ("*.cuh", "*.h", "*.hpp"):
            for f in Path(d).glob(ext):
                m = max(m, f.stat().st_mtime)
    return m


def _compile(cmd, src, obj, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compilation of {src} failed:\n{r.stdout}\n{r.stderr}")
    return obj


def build(verbose: bool = False, force: bool = False) -> None:
    LIBDIR.mkdir(parents=True, exist_ok=True)
    OBJDIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime([CSRC, CSRC / "rt"])
    jobs = []
    cu_objs, cpp_objs = [], []
    for src in sorted(CSRC.glob("*.cu")):
        obj = OBJDIR / (src.stem + ".o")
        cu_objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            jobs.append(([_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], src, obj))
    for src in sorted((CSRC / "rt").glob("*.cpp")):
        obj = OBJDIR / ("rt_" + src.stem + ".o")
        cpp_objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            jobs.append((["g++", *CXX_FLAGS, "-I", str(CSRC), "-I", "/usr/local/cuda/include", "-c", str(src), "-o", str(obj)], src, obj))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 4)) as ex:
            list(ex.map(lambda j: _compile(j[0], j[1], j[2], verbose), jobs))
    klib = LIBDIR / "libllmq_b200_kernels.so"
    if cu_objs and (force or jobs or not klib.exists()):
        cmd = [_nvcc(), "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(klib), *map(str, cu_objs)]
        _compile(cmd, "link kernels", klib, verbose)
    rlib = LIBDIR / "libllmq_b200_rt.so"
    if cpp_objs and (force or jobs or not rlib.exists()):
        cmd = ["g++", "-shared", "-pthread", "-o", str(rlib), *map(str, cpp_objs),
               "-L/usr/local/cuda/lib64", "-lcudart_static", "-ldl", "-lrt"]
        _compile(cmd, "link runtime", rlib, verbose)


def build_tests(verbose: bool = False) -> Path:
    """Native unit-test executable ``build/test_kernels`` (``csrc/tests/test_kernels.cu``), linked against the kernels library."""
    build(verbose=verbose)
    exe = PKG.parent / "build" / "test_kernels"
    src = CSRC / "tests" / "test_kernels.cu"
    klib = LIBDIR / "libllmq_b200_kernels.so"
    if not exe.exists() or exe.stat().st_mtime < max(src.stat().st_mtime, klib.stat().st_mtime):
        cmd = [_nvcc(), "-gencode", "arch=compute_100a,code=sm_100a", "-O2", "-std=c++17", str(src), "-o", str(exe),
               "-L", str(LIBDIR), "-lllmq_b200_kernels", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../llmq_b200/lib"]
        _compile(cmd, src, exe, verbose)
    return exe


if __name__ == "__main__":
    if "--tests" in sys.argv:
        print("built:", build_tests(verbose="-v" in sys.argv))
        sys.exit(0)
    build(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built:", *(p.name for p in LIBDIR.glob("*.so")))
