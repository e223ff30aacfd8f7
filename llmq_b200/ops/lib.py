"""ctypes loader for the in-tree native libraries.

The kernels library is required on any machine with a CUDA device: :func:`kernels` raises a
``RuntimeError`` instead of silently falling back when the shared object is missing, so a GPU run
can never pass on a PyTorch fallback by accident.
"""
from __future__ import annotations

import ctypes
import os
import threading
from pathlib import Path

import torch

_LIBDIR = Path(os.environ.get("LLMQ_LIB_DIR") or (Path(__file__).resolve().parent.parent / "lib"))      # LLMQ_LIB_DIR: another build of the libraries
_lock = threading.Lock()
_kernels = None
_rt = None

DT_BF16, DT_E4M3, DT_E5M2, DT_FP32, DT_FP16, DT_INT32, DT_INT8 = range(7)

_TORCH2CODE = {
    torch.bfloat16: DT_BF16,
    torch.float8_e4m3fn: DT_E4M3,
    torch.float8_e5m2: DT_E5M2,
    torch.float32: DT_FP32,
    torch.float16: DT_FP16,
    torch.int32: DT_INT32,
    torch.int8: DT_INT8,
}


def dtype_code(dt: torch.dtype) -> int:
    try:
        return _TORCH2CODE[dt]
    except KeyError:
        raise TypeError(f"unsupported dtype {dt}") from None


def _load(name: str):
    path = _LIBDIR / name
    if not path.exists():
        raise RuntimeError(
            f"native library {path} is missing; run `python -m llmq_b200.build` (needs nvcc, no GPU required)")
    return ctypes.CDLL(str(path))


def kernels():
    """Returns the CUDA kernels library (loads it on first use)."""
    global _kernels
    if _kernels is None:
        with _lock:
            if _kernels is None:
                _kernels = _load("libllmq_b200_kernels.so")
    return _kernels


def runtime():
    """Returns the host runtime library (data loader, safetensors writer, arena)."""
    global _rt
    if _rt is None:
        with _lock:
            if _rt is None:
                _rt = _load("libllmq_b200_rt.so")
    return _rt


def have_kernels() -> bool:
    return (_LIBDIR / "libllmq_b200_kernels.so").exists()


def ptr(t):
    """Device/host address of a tensor (``None`` -> NULL)."""
    if t is None:
        return ctypes.c_void_p(0)
    return ctypes.c_void_p(t.data_ptr())


def stream_ptr(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return ctypes.c_void_p(s.cuda_stream)


class KernelError(RuntimeError):
    pass


# Number of device kernels launched through this module (each entry point knows how many it launches).
_EXTRA_LAUNCHES = {"rmsnorm_backward": 1, "bias_backward": 1, "attention_backward": 2, "encoder_backward": 1}
launch_count = 0


def check(rc: int, what: str):
    global launch_count
    if rc != 0:
        raise KernelError(f"{what} failed with code {rc}")
    launch_count += 1 + _EXTRA_LAUNCHES.get(what, 0)
