"""Every kernel as a ``torch.library`` custom op (namespace ``llmq_b200``), the counterpart of the reference's
``pyllmq.kernels`` (src/binding/python/kernels.py:18-240): out-parameter style, tensors are mutated in place, so
the ops compose with ``torch.compile`` graphs and profilers while the hot path stays the hand-written kernels.

Ops launch on the current CUDA stream (the reference passes a raw stream handle instead).  ``matmul`` needs no
cuBLAS handle or workspace: it is the in-tree tcgen05 GEMM.
"""
from __future__ import annotations

from typing import Optional

import torch

from .ops import kernels as K

_op = torch.library.custom_op
T = torch.Tensor


def get_rmsnorm_backward_scratch_size(channels: int, device="cuda") -> int:
    return K.rmsnorm_backward_scratch_elems(channels, device) * 4


def get_bias_backward_scratch_size(dtype: torch.dtype, OC: int) -> int:
    return 64 * OC * 4


def get_qknorm_backward_scratch_size(Nq: int, Nkv: int, HeadDim: int, dtype: torch.dtype = torch.bfloat16) -> int:
    return 128 * 2 * HeadDim * 4


@_op("llmq_b200::encoder_forward", mutates_args=("out",))
def encoder_forward(out: T, inp: T, wte: T) -> None:
    K.encoder_forward(out, inp, wte)


@_op("llmq_b200::encoder_backward", mutates_args=("dwte",))
def encoder_backward(dwte: T, dout: T, inp: T) -> None:
    K.encoder_backward(dwte, dout, inp)


@_op("llmq_b200::rmsnorm_forward", mutates_args=("out", "rms", "absmax"))
def rmsnorm_forward(out: T, rms: T, inp: T, weight: T, absmax: Optional[T], epsilon: float) -> None:
    K.rmsnorm_forward(out, rms, inp, weight, epsilon, absmax=absmax)


@_op("llmq_b200::fused_residual_rmsnorm_forward", mutates_args=("residual", "normed", "rrms", "absmax"))
def fused_residual_rmsnorm_forward(residual: T, normed: T, rrms: T, inp1: T, inp2: T, weight: T, absmax: Optional[T], epsilon: float) -> None:
    K.rmsnorm_forward(normed, rrms, inp1, weight, epsilon, residual_out=residual, inp2=inp2, absmax=absmax)


@_op("llmq_b200::rmsnorm_backward", mutates_args=("dinp", "dweight", "scratch", "absmax"))
def rmsnorm_backward(dinp: T, dweight: T, scratch: T, dout: T, inp: T, weight: T, rstd: T, absmax: Optional[T]) -> None:
    """``dinp`` holds the upstream residual gradient on entry and the sum on exit."""
    K.rmsnorm_backward(dinp, dweight, scratch, dout, inp, weight, rstd, absmax=absmax)


@_op("llmq_b200::rope_forward", mutates_args=("out", "absmax"))
def rope_forward(out: T, x: T, freqs: T, absmax: Optional[T], Nq: int, Nkv: int) -> None:
    K.rope(out, x, freqs, Nq, Nkv, absmax=absmax)


@_op("llmq_b200::rope_backward", mutates_args=("dinp", "absmax"))
def rope_backward(dinp: T, dout: T, freqs: T, absmax: Optional[T], Nq: int, Nkv: int) -> None:
    K.rope(dinp, dout, freqs, Nq, Nkv, backward=True, absmax=absmax)


@_op("llmq_b200::qk_norm_forward", mutates_args=("out", "r_rms"))
def qk_norm_forward(out: T, r_rms: T, inp: T, q_weight: T, k_weight: T, epsilon: float, Nq: int, Nkv: int) -> None:
    K.qk_norm_forward(out, r_rms, inp, q_weight, k_weight, epsilon, Nq, Nkv)


@_op("llmq_b200::qk_norm_backward", mutates_args=("dinp", "dq_wgt", "dk_wgt", "scratch"))
def qk_norm_backward(dinp: T, dq_wgt: T, dk_wgt: T, scratch: T, dout: T, inp: T, q_weight: T, k_weight: T, r_rms: T, Nq: int, Nkv: int,
                     accumulate: bool = False) -> None:
    K.qk_norm_backward(dinp, dq_wgt, dk_wgt, scratch, dout, inp, q_weight, k_weight, r_rms, Nq, Nkv, accumulate)


@_op("llmq_b200::swiglu_forward", mutates_args=("out", "absmax"))
def swiglu_forward(out: T, inp: T, absmax: Optional[T]) -> None:
    K.swiglu_forward(out, inp, absmax=absmax)


@_op("llmq_b200::swiglu_forward_quant", mutates_args=("out", "scale"))
def swiglu_forward_quant(out: T, scale: T, inp: T, absmax: T) -> None:
    K.swiglu_forward(None, inp, q_out=out, known_absmax=absmax, q_scale=scale)


@_op("llmq_b200::swiglu_backward", mutates_args=("dinp", "absmax"))
def swiglu_backward(dinp: T, dout: T, inp: T, absmax: Optional[T]) -> None:
    K.swiglu_backward(dinp, dout, inp, absmax=absmax)


@_op("llmq_b200::attention_forward", mutates_args=("out", "stats"))
def attention_forward(out: T, stats: T, qkv: T, Nq: int, Nkv: int) -> None:
    K.attention_forward(out, stats, qkv, Nq, Nkv)


@_op("llmq_b200::attention_backward", mutates_args=("dqkv", "scratch"))
def attention_backward(dqkv: T, scratch: T, stats: T, out: T, dout: T, qkv: T, Nq: int, Nkv: int) -> None:
    K.attention_backward(dqkv, scratch, dout, out, stats, qkv, Nq, Nkv)


@_op("llmq_b200::fused_classifier", mutates_args=("logits", "losses", "lse"))
def fused_classifier(logits: T, losses: T, lse: T, dloss: float, targets: T, z_reg: float = 0.0, write_dlogits: bool = True) -> None:
    K.fused_classifier(logits, losses, lse, targets, dloss, z_reg, write_dlogits)


@_op("llmq_b200::grouped_loss_sum", mutates_args=("out",))
def grouped_loss_sum(out: T, per_token_loss: T) -> None:
    K.grouped_loss_sum(out, per_token_loss)


@_op("llmq_b200::matmul", mutates_args=("c", "absmax"))
def matmul(c: T, a: T, b: T, bias: Optional[T], scale_a: Optional[T], scale_b: Optional[T], absmax: Optional[T], mode: str = "TN",
           accumulate: bool = False) -> None:
    """c[M,N] (+)= op(a) @ op(b)^T.  ``mode`` names how the operands are stored: first letter for ``a`` ("T": [M,K]
    K contiguous, "N": [K,M]), second for ``b`` ("N": [N,K] K contiguous, "T": [K,N]) - i.e. "TN" is the plain
    ``a @ b.T`` of two row-major matrices."""
    K.gemm(c, a, b, a_mn=(mode[0] == "N"), b_mn=(mode[1] == "T"), bias=bias, accumulate=accumulate, scale_a=scale_a, scale_b=scale_b,
           absmax=absmax)


@_op("llmq_b200::matmul_mx", mutates_args=("c", "absmax"))
def matmul_mx(c: T, a: T, a_scales: T, b: T, b_scales: T, bias: Optional[T], absmax: Optional[T], accumulate: bool = False) -> None:
    """c[M,N] (+)= dq(a)[M,K] @ dq(b)[N,K]^T with block-scaled e4m3 operands (one power-of-two scale per 32 elements along K) from
    ``quantize_mx``.  No counterpart in the reference, whose fp8 matmuls are per-tensor scaled."""
    K.gemm_mx(c, a, a_scales, b, b_scales, bias=bias, accumulate=accumulate, absmax=absmax)


@_op("llmq_b200::quantize_mx", mutates_args=("out", "scales"))
def quantize_mx(out: T, scales: T, x: T, transpose: bool = False, operand: str = "a") -> None:
    """Block-scaled e4m3 form of bf16 ``x[R, C]``: along the rows, or (``transpose``) along the columns as ``out[C, R]``.
    ``scales`` holds ``mx_scale_bytes`` bytes in the GEMM's tiled layout for its ``a`` or ``b`` side."""
    K.quantize_mx(x, transpose=transpose, operand=operand, q_out=out, sf_out=scales)


def mx_scale_bytes(rows: int, k: int, operand: str = "a") -> int:
    return K.mx_sf_bytes(rows, k, K.MX_TILE_A if operand == "a" else K.MX_TILE_B)


@_op("llmq_b200::backward_bias", mutates_args=("dbias", "dbias_buffer"))
def backward_bias(dbias: T, dout: T, scale_a: Optional[T], scale_b: Optional[T], dbias_buffer: T, accumulate: bool = True) -> None:
    K.bias_backward(dbias, dout, dbias_buffer, scale_a=scale_a, scale_b=scale_b, accumulate=accumulate)


@_op("llmq_b200::abs_max", mutates_args=("scale",))
def abs_max(scale: T, x: T) -> None:
    K.abs_max(scale, x)


@_op("llmq_b200::quantize_with_abs_max", mutates_args=("out", "scale"))
def quantize_with_abs_max(out: T, scale: T, x: T, abs_max: T) -> None:
    K.quantize(out, scale, x, abs_max)


@_op("llmq_b200::quantize_and_transpose_with_abs_max", mutates_args=("out", "scale"))
def quantize_and_transpose_with_abs_max(out: T, scale: T, x: T, abs_max: T) -> None:
    K.transpose(out, x, absmax=abs_max, scale_out=scale)


@_op("llmq_b200::transpose", mutates_args=("dst",))
def transpose(dst: T, src: T) -> None:
    K.transpose(dst, src)


@_op("llmq_b200::vector_add_sr", mutates_args=("dest",))
def vector_add_sr(dest: T, left: T, right: T, scale: float, seed: int) -> None:
    K.vector_add_sr(dest, left, right, scale, seed)


@_op("llmq_b200::vector_reduce_sr", mutates_args=("dest",))
def vector_reduce_sr(dest: T, src: T, scale: float, n_shards: int, skip: int, accumulate: bool, seed: int) -> None:
    K.vector_reduce_sr(dest, src, scale, n_shards, skip=skip, accumulate=accumulate, seed=seed)


@_op("llmq_b200::fill_normal", mutates_args=("dst",))
def fill_normal(dst: T, mean: float, std: float, seed: int, subsequence: int = 0) -> None:
    K.fill_normal(dst, mean, std, seed, subsequence)


@_op("llmq_b200::fill_constant", mutates_args=("dst",))
def fill_constant(dst: T, value: float) -> None:
    K.fill(dst, value)


@_op("llmq_b200::convert_dtype", mutates_args=("dst",))
def convert_dtype(dst: T, src: T) -> None:
    K.convert(dst, src)


@_op("llmq_b200::global_norm_squared", mutates_args=("out",))
def global_norm_squared(out: T, values: T) -> None:
    K.norm_squared(out, values)


@_op("llmq_b200::global_norm_finish", mutates_args=("io", "partials"))
def global_norm_finish(io: T, partials: T, grad_clip: float) -> None:
    K.deterministic_sum(io[0:1], partials)
    K.norm_finish(io, grad_clip)


@_op("llmq_b200::adamw_update", mutates_args=("params", "m", "v", "m_scales", "abs_max"))
def adamw_update_impl(params: T, grads: T, m: T, v: T, m_scales: Optional[T], abs_max: Optional[T], grad_scale: Optional[T], lr: float,
                      beta1: float, beta2: float, step: int, eps: float, weight_decay: float, seed: int) -> None:
    K.adamw(params, grads, m, v, lr=lr, beta1=beta1, beta2=beta2, step=step, eps=eps, weight_decay=weight_decay, grad_scale=grad_scale,
            absmax=abs_max, m_scales=m_scales, seed=seed)


def adamw_update(params, grads, m, v, lr, beta1, beta2, step, eps, weight_decay, grad_scale=None, m_scales=None, abs_max=None, seed=0):
    adamw_update_impl(params, grads, m, v, m_scales, abs_max, grad_scale, lr, beta1, beta2, step, eps, weight_decay, seed)
