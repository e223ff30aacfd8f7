"""NVTX ranges for timeline tools (role of ``NvtxRange`` / ``NVTX_RANGE_FN`` in the reference, ``utils.h:97-103``): the
step phases, every layer, weight gathers, the LM head, recomputation and offload transfers are named with the
reference's range names.  Host-side markers only; without a profiler attached they cost about a microsecond each.
``LLMQ_NVTX=0`` switches them off; they are off on CPU tensors and switch themselves off if the first call fails."""
from __future__ import annotations

import contextlib
import os

import torch

_state = {"on": os.environ.get("LLMQ_NVTX", "1") != "0"}


def _backend():
    return torch.cuda.nvtx


def push(name: str, device=None) -> bool:
    """Opens a range; returns whether one was opened (pass that to :func:`pop`)."""
    if not _state["on"] or (device is not None and torch.device(device).type != "cuda"):
        return False
    try:
        _backend().range_push(name)
        return True
    except Exception:
        _state["on"] = False            # no NVTX in this build: stay silent from here on
        return False


def pop(opened: bool = True) -> None:
    if opened and _state["on"]:
        try:
            _backend().range_pop()
        except Exception:
            _state["on"] = False


@contextlib.contextmanager
def range(name: str, device=None):
    opened = push(name, device)
    try:
        yield
    finally:
        pop(opened)
