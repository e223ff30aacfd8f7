#!/usr/bin/env python
"""Builds the UNMODIFIED reference (IST-DASLab/llmq) from its sources, offline, for the reference arm of bench.py.

The reference's CMake project downloads nlohmann-json, cudnn-frontend, CLI11, nanobind, fmt and Catch2 with
FetchContent (CMakeLists.txt:22-70), which cannot work without a network.  Everything its library target
``llmq-common`` needs (CMakeLists.txt:136-190) is on disk, though: cudnn_frontend.h with its bundled
nlohmann/json.hpp, the header-only fmt that ships with torch, nccl.h, cudnn.h, cuBLASLt and NVML.  CLI11, nanobind
and Catch2 are only used by train.cpp, the Python binding and the unit tests, none of which the benchmark arm needs.

This script compiles every source of ``llmq-common`` (same list, same definitions: USE_THREADS=1, no MPI, no cuFile,
NVML on; Release flags) for sm_100a into ``baseline/_ref/libllmq-common.so`` and links ``baseline/ref_harness.cpp``
(a small ``main`` over the reference's public C++ API, the loop of train.cpp:512-590) against it as
``baseline/_ref/ref_bench``.  No reference file is edited or copied into the repository.

    python baseline/build_ref.py [--reference /path/to/llmq] [--jobs N]
"""
import argparse
import concurrent.futures as cf
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")

SOURCES = """
src/utilities/safetensors.cpp src/utilities/cu_file_fallback.cpp src/utilities/gpu_info_nvml.cpp
src/utilities/allocator.cpp src/utilities/lazy_allocator.cpp src/utilities/utils.cpp src/utilities/comm.cpp
src/utilities/tensor.cpp src/utilities/sol.cpp src/utilities/dtype.cpp src/utilities/stack.cpp
src/training/adamw_optimizer.cpp src/training/dataloader.cpp src/training/logging.cpp src/training/checkpoint.cpp
src/training/model.cpp src/training/gradients.cpp src/training/transformer_config.cpp
src/models/llama_run_state.cpp src/models/llama_model.cpp src/models/llama_weights.cpp src/models/llama_gradients.cpp
src/models/llama_optimizer.cpp
src/kernels/kernels.cpp src/kernels/encoder.cu src/kernels/matmul.cpp src/kernels/swiglu.cu src/kernels/rope.cu
src/kernels/rmsnorm.cu src/kernels/cudnn_att.cpp src/kernels/quant.cu src/kernels/global_norm.cu src/kernels/bias.cu
src/kernels/adamw.cu src/kernels/attention.cu src/kernels/fused_classifier.cu src/kernels/fused_classifier_tma.cu
src/kernels/transpose.cu src/kernels/vector_add.cu src/kernels/random.cu src/kernels/fill.cu src/kernels/convert.cu
src/kernels/gemm_mma.cu src/kernels/qk_norm.cu
""".split()


def find_first(paths):
    for p in paths:
        if os.path.exists(p):
            return p
    raise FileNotFoundError(paths)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("LLMQ_REFERENCE", "/root/reference"))
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 8)
    args = ap.parse_args()
    ref = os.path.abspath(args.reference)
    site = sysconfig.get_paths()["purelib"]
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    obj = os.path.join(OUT, "obj")
    inc = os.path.join(OUT, "include")
    os.makedirs(obj, exist_ok=True)
    os.makedirs(inc, exist_ok=True)
    # An include folder with just the three third-party header trees, so nothing else of torch's include
    # directory can shadow a system header.
    links = {
        "fmt": find_first([os.path.join(site, "torch/include/fmt")]),
        "cudnn_frontend": find_first([os.path.join(site, "include/cudnn_frontend")]),
        "cudnn_frontend.h": find_first([os.path.join(site, "include/cudnn_frontend.h")]),
    }
    for name, target in links.items():
        dst = os.path.join(inc, name)
        if os.path.islink(dst):
            os.unlink(dst)
        os.symlink(target, dst)
    # nlohmann-json exists on disk only as the single header bundled with cudnn-frontend; the reference also includes
    # <nlohmann/json_fwd.hpp> (forward declarations), which the single header contains: a one-line forwarding header
    # in the build folder stands in for it.
    nl = os.path.join(inc, "nlohmann")
    if os.path.islink(nl):
        os.unlink(nl)
    os.makedirs(nl, exist_ok=True)
    dst = os.path.join(nl, "json.hpp")
    if os.path.islink(dst):
        os.unlink(dst)
    os.symlink(find_first([os.path.join(site, "include/cudnn_frontend/thirdparty/nlohmann/json.hpp")]), dst)
    with open(os.path.join(nl, "json_fwd.hpp"), "w") as f:
        f.write("#pragma once\n#include \"json.hpp\"\n")
    for h in os.listdir(os.path.join(site, "include")):
        if h.startswith("cudnn_") and h.endswith(".h"):
            dst = os.path.join(inc, h)
            if os.path.islink(dst):
                os.unlink(dst)
            os.symlink(os.path.join(site, "include", h), dst)
    # cuDNN, NCCL and cuBLASLt: the Python environment's copies first, as the reference's own wheel resolves them
    # (its RPATH is $ORIGIN/../nvidia/{nccl,cudnn,cuda_runtime,cublas}/lib, CMakeLists.txt:211-218).  The system cuDNN
    # (9.10) is too old for the deterministic SDPA backward the reference asks for on Blackwell (needs >= 9.18).
    nv = os.path.join(site, "nvidia")
    cudnn_inc = os.path.dirname(find_first([os.path.join(nv, "cudnn/include/cudnn.h"), "/usr/include/x86_64-linux-gnu/cudnn.h", "/usr/include/cudnn.h"]))
    nccl_inc = os.path.dirname(find_first([os.path.join(nv, "nccl/include/nccl.h"), "/usr/include/nccl.h"]))
    env_libs = [d for d in (os.path.join(nv, "cudnn/lib"), os.path.join(nv, "nccl/lib"), os.path.join(nv, "cublas/lib"),
                            os.path.join(nv, "cuda_runtime/lib")) if os.path.isdir(d)]
    common = [f"-I{ref}/src", f"-I{inc}", f"-I{cudnn_inc}", f"-I{nccl_inc}", f"-I{cuda}/include",
              "-DFMT_HEADER_ONLY=1", "-DUSE_THREADS=1", "-DNDEBUG"]
    nvcc = [os.path.join(cuda, "bin/nvcc"), "-std=c++20", "-O3", "-gencode", "arch=compute_100a,code=sm_100a",
            "--expt-relaxed-constexpr", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-pthread"] + common
    gxx = ["g++", "-std=c++20", "-O3", "-fPIC", "-pthread"] + common

    def compile_one(src):
        path = os.path.join(ref, src)
        out = os.path.join(obj, src.replace("/", "_") + ".o")
        if os.path.exists(out) and os.path.getmtime(out) > os.path.getmtime(path):
            return src, 0, ""
        cmd = (nvcc if src.endswith(".cu") else gxx) + ["-c", path, "-o", out]
        r = subprocess.run(cmd, capture_output=True, text=True)
        return src, r.returncode, r.stdout + r.stderr

    failed = False
    with cf.ThreadPoolExecutor(args.jobs) as ex:
        for src, rc, log in ex.map(compile_one, SOURCES):
            print(("ok   " if rc == 0 else "FAIL ") + src, flush=True)
            if rc != 0:
                failed = True
                print(log[-4000:])
    if failed:
        return 1
    objs = [os.path.join(obj, s.replace("/", "_") + ".o") for s in SOURCES]
    lib = os.path.join(OUT, "libllmq-common.so")
    libdirs = [f"-L{d}" for d in env_libs] + [f"-L{cuda}/lib64", f"-L{cuda}/lib64/stubs", "-L/usr/lib/x86_64-linux-gnu"]
    rpaths = ["-Xlinker", "-rpath," + ":".join(env_libs + [f"{cuda}/lib64"])]
    link = [os.path.join(cuda, "bin/nvcc"), "-shared", "--cudart", "shared", "-Wno-deprecated-gpu-targets", "-o", lib] + objs + libdirs + \
           rpaths + ["-l:libcudnn.so.9", "-l:libnccl.so.2", "-l:libcublasLt.so.12", "-l:libcublas.so.12", "-lnvidia-ml", "-l:libcudart.so.12"]
    r = subprocess.run(link, capture_output=True, text=True)
    print(r.stdout + r.stderr)
    if r.returncode:
        return r.returncode
    exe = os.path.join(OUT, "ref_bench")
    r = subprocess.run(gxx + [os.path.join(HERE, "ref_harness.cpp"), "-o", exe, f"-L{OUT}", "-lllmq-common",
                              "-Wl,-rpath,$ORIGIN"] + libdirs + ["-Wl,-rpath," + ":".join(env_libs + [f"{cuda}/lib64"]), "-lnvidia-ml", "-l:libcudart.so.12", "-l:libnccl.so.2", "-lpthread"],
                       capture_output=True, text=True)
    print(r.stdout + r.stderr)
    if r.returncode == 0:
        print("built", exe)
    return r.returncode


if __name__ == "__main__":
    sys.exit(main())
