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


# ---- the reference's argument lists for the calls whose extra arguments have no job here (library handles, host-side
# bucket tables, workspaces).  Each forwards to the op of the same name in ``llmq_b200.kernels_api``.
import llmq_b200.kernels_api as _api


def encoder_forward(out: torch.Tensor, inp: torch.Tensor, wte: torch.Tensor, wpe: Optional[torch.Tensor] = None, stream: int = 0) -> None:
    """``out = wte[inp]`` (+ ``wpe`` per position, which the Llama / Qwen2 models never pass)."""
    _api.encoder_forward(out, inp, wte)
    if wpe is not None:
        out.add_(wpe.to(out.dtype).reshape(1, *wpe.shape))


def encoder_backward(dwte: torch.Tensor, scratch: Optional[torch.Tensor], workload_indices: Optional[torch.Tensor],
                     bucket_info: Optional[torch.Tensor], dout: torch.Tensor, inp: torch.Tensor, inputs_cpu: Optional[torch.Tensor] = None,
                     seed: int = 0, stream: int = 0, sync_event: int = 0, copy_stream: int = 0) -> None:
    """Deterministic embedding gradient.  The bucket tables, the host copy of the tokens and the copy stream exist in the
    reference for its host-side bucket sort; here the sort runs on the device, so they are ignored."""
    _api.encoder_backward(dwte, dout, inp)


def rmsnorm_backward(dinp: torch.Tensor, dweight: torch.Tensor, scratch: torch.Tensor, dresidual: torch.Tensor, dout: torch.Tensor,
                     inp: torch.Tensor, weight: torch.Tensor, rstd: torch.Tensor, absmax: Optional[torch.Tensor] = None, stream: int = 0) -> None:
    """``dinp = dresidual + d(rmsnorm)`` (``dresidual`` may be ``dinp`` itself)."""
    if dresidual.data_ptr() != dinp.data_ptr():
        dinp.copy_(dresidual)
    _api.rmsnorm_backward(dinp, dweight, scratch, dout, inp, weight, rstd, absmax)


def qk_norm_backward(dinp: torch.Tensor, dq_wgt: torch.Tensor, dk_wgt: torch.Tensor, scratch: torch.Tensor, dout: torch.Tensor, inp: torch.Tensor,
                     q_wgt: torch.Tensor, k_wgt: torch.Tensor, rstd: torch.Tensor, abs_max: Optional[torch.Tensor] = None, Nq: int = 0, Nkv: int = 0,
                     stream: int = 0) -> None:
    _api.qk_norm_backward(dinp, dq_wgt, dk_wgt, scratch, dout, inp, q_wgt, k_wgt, rstd, Nq, Nkv)
    if abs_max is not None:
        _api.abs_max(abs_max, dinp)


def _float_view(workspace: Optional[torch.Tensor], elems: int, like: torch.Tensor) -> torch.Tensor:
    if workspace is not None and workspace.is_contiguous() and workspace.device == like.device and workspace.numel() * workspace.element_size() >= 4 * elems:
        return workspace.view(torch.uint8)[: 4 * elems].view(torch.float32)
    return torch.empty(elems, dtype=torch.float32, device=like.device)


def attention_forward(out: torch.Tensor, stats: torch.Tensor, inp: torch.Tensor, workspace: Optional[torch.Tensor] = None, cudnn_handle: int = 0,
                      Hq: int = 0, Hkv: int = 0, stream: int = 0) -> None:
    """Causal GQA attention on packed ``inp`` [B, T, Hq + 2 Hkv, HS]; the in-tree kernel needs neither workspace nor handle."""
    _api.attention_forward(out, stats, inp, Hq, Hkv)


def attention_backward(dqkv: torch.Tensor, stats: torch.Tensor, out: torch.Tensor, dout: torch.Tensor, qkv: torch.Tensor,
                       workspace: Optional[torch.Tensor] = None, cudnn_handle: int = 0, Hq: int = 0, Hkv: int = 0, stream: int = 0) -> None:
    """The only scratch is one float per (batch, head, position); it is taken from ``workspace`` when that is large enough."""
    _api.attention_backward(dqkv, _float_view(workspace, stats.numel(), qkv), stats, out, dout, qkv, Hq, Hkv)
