"""``pyllmq.kernels``: the torch custom ops of ``llmq_b200.kernels_api``, plus the three names whose signature in the
reference carries a cuBLASLt handle (``binding/python/kernels.py:120-134`` there): there is no library handle here, the
GEMMs are the in-tree tcgen05 kernels, so the handle is a dummy and the workspace argument is ignored."""
from typing import Optional

import torch

from llmq_b200.kernels_api import *  # noqa: F401,F403
from llmq_b200.ops import kernels as _K

MM_TT, MM_TN, MM_NT, MM_NN = 0, 1, 2, 3        # the reference's EMMTranspose values


def create_cublas_handle() -> int:
    """No library handle exists; the value only has to be passed back to ``matmul`` / ``destroy_cublas_handle``."""
    return 0


def destroy_cublas_handle(handle: int) -> None:
    return None


def matmul(c: torch.Tensor, a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor], scale_a: Optional[torch.Tensor],
           scale_b: Optional[torch.Tensor], cublaslt_handle: int = 0, workspace: Optional[torch.Tensor] = None, mode: int = MM_NT,
           accumulate: bool = False, stream: int = 0) -> None:
    """The reference's call: ``c (+)= op(a) @ op(b) (+ bias)`` in row-major terms, where ``mode`` (TT, TN, NT, NN = 0..3)
    says which of ``a`` / ``b`` is stored transposed; ``scale_a * scale_b`` de-quantises fp8 operands.  Runs on the
    current stream (``stream`` is accepted for compatibility)."""
    if mode not in (MM_TT, MM_TN, MM_NT, MM_NN):
        raise ValueError("Invalid mode")
    a_t, b_t = mode in (MM_TT, MM_TN), mode in (MM_TT, MM_NT)
    _K.gemm(c, a, b, a_mn=a_t, b_mn=not b_t, bias=bias, accumulate=accumulate, scale_a=scale_a, scale_b=scale_b)
