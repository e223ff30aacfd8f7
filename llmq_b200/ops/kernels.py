"""Tensor-level entry points of every kernel.

Each function works on pre-allocated ``torch`` tensors (no allocation on the hot path) and launches
on the current CUDA stream.  CUDA tensors always go to the hand-written sm_100a kernels of
``libllmq_b200_kernels.so``; a missing library is an error, never a silent fallback.  CPU tensors take
a plain PyTorch implementation of the same mathematics, which is what the CPU test-suite, the gloo
multi-rank tests and the numerics oracles run on.

The set of operations mirrors the kernel API of the reference (src/kernels/kernels.h:25-295).
"""
from __future__ import annotations

import ctypes
import os
import math
from typing import Optional

import torch

from . import lib as L

F8 = torch.float8_e4m3fn
F8_E5 = torch.float8_e5m2
_FP8_MAX = {F8: 448.0, F8_E5: 57344.0}

_state = {}


def _dev_state(device):
    device = torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    st = _state.get(idx)
    if st is None:
        with torch.cuda.device(idx):
            props = torch.cuda.get_device_properties(idx)
            st = {
                "sms": props.multi_processor_count,
                "status": torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}"),
                # fp32 scratch of the split-K GEMM path (small outputs with a long K: weight gradients of small models)
                "splitk_ws": torch.empty(SPLITK_WS_FLOATS, dtype=torch.float32, device=f"cuda:{idx}"),
                "splitk_tid": None,
            }
        _state[idx] = st
    return st


SPLITK_WS_FLOATS = 16 << 20


def _bind_splitk(st) -> None:
    """The workspace is registered per calling thread (rank threads each drive their own device)."""
    import threading
    tid = threading.get_ident()
    if st["splitk_tid"] != tid:
        ws = st["splitk_ws"] if os.environ.get("LLMQ_GEMM_SPLITK", "1") != "0" else None
        L.kernels().llmq_gemm_set_splitk_workspace(L.ptr(ws), ctypes.c_longlong(0 if ws is None else ws.numel()))
        st["splitk_tid"] = tid


def num_sms(device) -> int:
    return _dev_state(device)["sms"]


def status_word(device) -> torch.Tensor:
    """Device word into which kernels OR an error code when one of their bounded waits runs out."""
    return _dev_state(device)["status"]


def check_status(device) -> None:
    """Raises if any kernel reported a timed-out wait since the last check (synchronises)."""
    st = _dev_state(device)["status"]
    v = int(st.item())
    if v != 0:
        st.zero_()
        raise L.KernelError(f"a device-side wait timed out (status 0x{v:x}); the step result is invalid")


_scratch_bufs = {}


def _scratch(tag: str, device, shape, dtype) -> torch.Tensor:
    """Device scratch per (tag, device, shape, dtype), allocated on first use (conversion paths of the fp32 model)."""
    key = (tag, str(device), tuple(shape), dtype)
    buf = _scratch_bufs.get(key)
    if buf is None:
        buf = _scratch_bufs[key] = torch.empty(tuple(shape), dtype=dtype, device=device)
    return buf


def _ll(v):
    return ctypes.c_longlong(int(v))


def _f(v):
    return ctypes.c_float(float(v))


def _is_f8(dt):
    return dt in (F8, F8_E5)


# =====================================================================================================
# GEMM
def gemm(out: torch.Tensor, a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         bias: Optional[torch.Tensor] = None, accumulate: bool = False, scale_a: Optional[torch.Tensor] = None,
         scale_b: Optional[torch.Tensor] = None, alpha: float = 1.0, absmax: Optional[torch.Tensor] = None,
         ready=None) -> None:
    """out[M,N] (+)= alpha * scale_a * scale_b * A @ B^T + bias.

    ``ready`` = (flag address, generation, rows per source rank, limit in seconds): the rows of the stored ``b`` are
    being written by peer GPUs (fused all-gather); the kernel's producer polls the flags tile by tile.

    ``a`` holds the logical [M,K] operand either as [M,K] (K-major) or, with ``a_mn``, as [K,M];
    likewise ``b`` holds logical [N,K] as [N,K] or, with ``b_mn``, as [K,N].  2-D, last dim contiguous.
    """
    M, N = out.shape
    K = a.shape[0] if a_mn else a.shape[1]
    assert (a.shape[1] if a_mn else a.shape[0]) == M, (a.shape, out.shape, a_mn)
    assert (b.shape == (K, N)) if b_mn else (b.shape == (N, K)), (b.shape, (N, K), b_mn)
    if out.is_cuda and a.dtype == torch.float32 and (a_mn or b_mn):
        # fp32 operands (tf32 MMA kind) are only fed K-major: transpose the other forms into scratch first
        assert a.is_contiguous() and b.is_contiguous()
        if a_mn:
            at = _scratch("gemm_a_T", a.device, (M, K), torch.float32)
            transpose(at, a)
            a, a_mn = at, False
        if b_mn:
            bt = _scratch("gemm_b_T", b.device, (N, K), torch.float32)
            transpose(bt, b)
            b, b_mn = bt, False
    if out.is_cuda:
        st = _dev_state(out.device)
        _bind_splitk(st)
        assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
        assert a.dtype == b.dtype or (_is_f8(a.dtype) and _is_f8(b.dtype)), (a.dtype, b.dtype)
        rflags, rgen, rrows, rlimit = ready if ready is not None else (0, 0, 0, 0.0)
        rc = L.kernels().llmq_gemm_ready(
            L.ptr(a), L.ptr(b), L.ptr(out), L.ptr(bias), M, N, K, L.dtype_code(a.dtype), L.dtype_code(b.dtype),
            int(a_mn), int(b_mn), _ll(a.stride(0)), _ll(b.stride(0)), _ll(out.stride(0)),
            0 if out.dtype == torch.bfloat16 else 1, 0 if (bias is None or bias.dtype == torch.bfloat16) else 1,
            int(accumulate), L.ptr(scale_a), L.ptr(scale_b), _f(alpha), L.ptr(absmax), L.ptr(st["status"]), st["sms"],
            ctypes.c_void_p(rflags), ctypes.c_uint(rgen), int(rrows), ctypes.c_double(rlimit), L.stream_ptr())
        L.check(rc, "gemm")
        return
    af = a.float().t() if a_mn else a.float()
    bf = b.float() if b_mn else b.float().t()
    r = af @ bf
    s = alpha
    if scale_a is not None:
        s = s * scale_a.float()
    if scale_b is not None:
        s = s * scale_b.float()
    r = r * s
    if bias is not None:
        r = r + bias.float()
    if accumulate:
        r = r + out.float()
    out.copy_(r.to(out.dtype))
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, out.float().abs().max().reshape_as(absmax)))


def gemm_swiglu_forward(up_out: torch.Tensor, act_out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, *,
                        scale_a: Optional[torch.Tensor] = None, scale_b: Optional[torch.Tensor] = None,
                        absmax: Optional[torch.Tensor] = None) -> None:
    """up_out[M, 2D] = a @ w^T (w rows = [up | gate]) and act_out[M, D] = up * gate * sigmoid(gate) from the same
    accumulator tile; ``absmax`` tracks act_out.  CUDA only (bf16 outputs, M >= 256, D a multiple of 128)."""
    M, D = act_out.shape
    st = _dev_state(a.device)
    rc = L.kernels().llmq_gemm_swiglu(L.ptr(a), L.ptr(w), L.ptr(up_out), L.ptr(act_out), 1, M, D, a.shape[1], L.dtype_code(a.dtype),
                                      L.dtype_code(w.dtype), 0, 0, _ll(a.stride(0)), _ll(w.stride(0)), L.ptr(scale_a), L.ptr(scale_b),
                                      _f(1.0), L.ptr(absmax), L.ptr(st["status"]), st["sms"], L.stream_ptr())
    L.check(rc, "gemm_swiglu_forward")


def gemm_swiglu_backward(up_inout: torch.Tensor, dout: torch.Tensor, w: torch.Tensor, *, scale_a: Optional[torch.Tensor] = None,
                         scale_b: Optional[torch.Tensor] = None, absmax: Optional[torch.Tensor] = None) -> None:
    """d(act) = dout[M, C] @ w[C, D] stays in the accumulator; up_inout[M, 2D] goes from [up | gate] to [d_up | d_gate]."""
    M, D2 = up_inout.shape
    st = _dev_state(dout.device)
    rc = L.kernels().llmq_gemm_swiglu(L.ptr(dout), L.ptr(w), None, L.ptr(up_inout), 2, M, D2 // 2, dout.shape[1], L.dtype_code(dout.dtype),
                                      L.dtype_code(w.dtype), 0, 1, _ll(dout.stride(0)), _ll(w.stride(0)), L.ptr(scale_a), L.ptr(scale_b),
                                      _f(1.0), L.ptr(absmax), L.ptr(st["status"]), st["sms"], L.stream_ptr())
    L.check(rc, "gemm_swiglu_backward")


def gemm_swiglu_supported(M: int, D: int, t: torch.Tensor) -> bool:
    return t.is_cuda and t.dtype == torch.bfloat16 and M >= 256 and D % 128 == 0


# =====================================================================================================
# Block-scaled (MX) e4m3: one UE8M0 scale per 32 elements of the contraction axis (csrc/quant_mx.cu, csrc/gemm_mx_tcgen05.cu)
MX_TILE_A, MX_TILE_B = 128, 224        # rows per scale-factor tile of the GEMM's A / B operand


def mx_sf_offsets(rows: int, K: int, tile_rows: int) -> torch.Tensor:
    """Byte offset of the scale of (row, 32-element block) in the tiled scale-factor buffer, as an int64 [rows, K/32] tensor."""
    chunks = (tile_rows + 127) // 128
    n_tiles = (rows + tile_rows - 1) // tile_rows
    r = torch.arange(rows).unsqueeze(1)
    kb = torch.arange(K // 32).unsqueeze(0)
    tile, rt = r // tile_rows, r % tile_rows
    rr = rt % 128
    return (((kb // 4) * n_tiles + tile) * chunks + rt // 128) * 512 + (rr % 32) * 16 + (rr // 32) * 4 + kb % 4


def mx_sf_bytes(rows: int, K: int, tile_rows: int) -> int:
    return (K // 128) * ((rows + tile_rows - 1) // tile_rows) * ((tile_rows + 127) // 128) * 512


def quantize_mx(x: torch.Tensor, *, transpose: bool = False, operand: str = "a", q_out: Optional[torch.Tensor] = None,
                sf_out: Optional[torch.Tensor] = None):
    """bf16 ``x[R, C]`` -> (e4m3 values, uint8 scale buffer) for :func:`gemm_mx`.  ``transpose`` quantises along the rows and
    returns the transposed matrix ``[C, R]`` (the operand of a GEMM that contracts over R); ``operand`` ("a" / "b") picks the
    scale-factor tiling of the GEMM side the result feeds.  The contraction length must be a multiple of 128."""
    R, C = x.shape
    rows, K = (C, R) if transpose else (R, C)
    tile = MX_TILE_A if operand == "a" else MX_TILE_B
    assert K % 128 == 0, "MX operands need a contraction length that is a multiple of 128"
    if q_out is None:
        q_out = torch.empty((rows, K), dtype=F8, device=x.device)
    if sf_out is None:
        sf_out = torch.empty(mx_sf_bytes(rows, K, tile), dtype=torch.uint8, device=x.device)
    assert q_out.shape == (rows, K) and q_out.is_contiguous() and sf_out.numel() >= mx_sf_bytes(rows, K, tile)
    if x.is_cuda:
        assert x.dtype == torch.bfloat16 and x.stride(1) == 1
        rc = L.kernels().llmq_quantize_mx(L.ptr(q_out), L.ptr(sf_out), L.ptr(x), _ll(R), _ll(C), _ll(x.stride(0)), int(transpose), tile,
                                          L.stream_ptr())
        L.check(rc, "quantize_mx")
        return q_out, sf_out
    xs = (x.t() if transpose else x).float().reshape(rows, K // 32, 32)
    amax = xs.abs().amax(-1)
    e = torch.where(amax > 0, torch.ceil(torch.log2(amax.double() / 448.0)).clamp(-127, 126), torch.full_like(amax, -127.0, dtype=torch.float64))
    q_out.copy_((xs * torch.exp2(-e).float().unsqueeze(-1)).clamp(-448, 448).reshape(rows, K).to(F8))
    sf_out.zero_()
    sf_out[mx_sf_offsets(rows, K, tile).reshape(-1)] = (e + 127).to(torch.uint8).reshape(-1)
    return q_out, sf_out


def quantize_mx_both(x: torch.Tensor, *, row_operand: str = "a", col_operand: str = "a", q_rows=None, sf_rows=None, q_cols=None, sf_cols=None):
    """Row form and column (transposed) form of ``x[R, C]`` from one pass over it: ``(q_rows[R, C], sf_rows, q_cols[C, R], sf_cols)``.
    R and C must be multiples of 128."""
    R, C = x.shape
    assert R % 128 == 0 and C % 128 == 0
    tr, tc = (MX_TILE_A if row_operand == "a" else MX_TILE_B), (MX_TILE_A if col_operand == "a" else MX_TILE_B)
    if q_rows is None:
        q_rows = torch.empty((R, C), dtype=F8, device=x.device)
    if q_cols is None:
        q_cols = torch.empty((C, R), dtype=F8, device=x.device)
    if sf_rows is None:
        sf_rows = torch.empty(mx_sf_bytes(R, C, tr), dtype=torch.uint8, device=x.device)
    if sf_cols is None:
        sf_cols = torch.empty(mx_sf_bytes(C, R, tc), dtype=torch.uint8, device=x.device)
    if x.is_cuda:
        assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and q_rows.is_contiguous() and q_cols.is_contiguous()
        rc = L.kernels().llmq_quantize_mx_both(L.ptr(q_rows), L.ptr(sf_rows), tr, L.ptr(q_cols), L.ptr(sf_cols), tc, L.ptr(x), _ll(R), _ll(C),
                                               _ll(x.stride(0)), L.stream_ptr())
        L.check(rc, "quantize_mx_both")
    else:
        quantize_mx(x, operand=row_operand, q_out=q_rows, sf_out=sf_rows)
        quantize_mx(x, transpose=True, operand=col_operand, q_out=q_cols, sf_out=sf_cols)
    return q_rows, sf_rows, q_cols, sf_cols


def dequantize_mx(q: torch.Tensor, sf: torch.Tensor, operand: str = "a") -> torch.Tensor:
    """fp32 values of a block-scaled operand (reference / debugging)."""
    rows, K = q.shape
    off = mx_sf_offsets(rows, K, MX_TILE_A if operand == "a" else MX_TILE_B).to(sf.device)
    e = sf[off.reshape(-1)].reshape(rows, K // 32).float() - 127.0
    return (q.float().reshape(rows, K // 32, 32) * torch.exp2(e).unsqueeze(-1)).reshape(rows, K)


def gemm_mx(out: torch.Tensor, a: torch.Tensor, a_sf: torch.Tensor, b: torch.Tensor, b_sf: torch.Tensor, *,
            bias: Optional[torch.Tensor] = None, accumulate: bool = False, alpha: float = 1.0,
            absmax: Optional[torch.Tensor] = None) -> None:
    """out[M, N] (+)= alpha * dq(a)[M, K] @ dq(b)[N, K]^T + bias with block-scaled e4m3 operands from :func:`quantize_mx`."""
    M, N = out.shape
    K = a.shape[1]
    assert a.shape == (M, K) and b.shape == (N, K) and K % 128 == 0
    if out.is_cuda:
        st = _dev_state(out.device)
        rc = L.kernels().llmq_gemm_mx(L.ptr(a), L.ptr(b), L.ptr(a_sf), L.ptr(b_sf), L.ptr(out), L.ptr(bias), M, N, K, _ll(a.stride(0)),
                                      _ll(b.stride(0)), _ll(out.stride(0)), 0 if out.dtype == torch.bfloat16 else 1,
                                      0 if (bias is None or bias.dtype == torch.bfloat16) else 1, int(accumulate), _f(alpha), L.ptr(absmax),
                                      L.ptr(st["status"]), st["sms"], L.stream_ptr())
        L.check(rc, "gemm_mx")
        return
    r = alpha * (dequantize_mx(a, a_sf, "a") @ dequantize_mx(b, b_sf, "b").t())
    if bias is not None:
        r = r + bias.float()
    if accumulate:
        r = r + out.float()
    out.copy_(r.to(out.dtype))
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, out.float().abs().max().reshape_as(absmax)))


# =====================================================================================================
# RMSNorm
def rmsnorm_forward(y: Optional[torch.Tensor], rstd: Optional[torch.Tensor], inp: torch.Tensor, weight: torch.Tensor, eps: float,
                    *, residual_out: Optional[torch.Tensor] = None, inp2: Optional[torch.Tensor] = None,
                    absmax: Optional[torch.Tensor] = None, q_out: Optional[torch.Tensor] = None,
                    known_absmax: Optional[torch.Tensor] = None, q_scale: Optional[torch.Tensor] = None) -> None:
    """(residual_out = inp + inp2;) y = T(x * rstd) * weight with x the (summed) input.

    ``q_out`` (e4m3) together with ``known_absmax`` emits the quantised result directly.
    """
    C = inp.shape[-1]
    rows = inp.numel() // C
    if inp.is_cuda:
        rc = L.kernels().llmq_rmsnorm_forward(
            L.ptr(residual_out), L.ptr(y), L.ptr(q_out), L.ptr(rstd), L.ptr(inp), L.ptr(inp2), L.ptr(weight), _f(eps), rows, C,
            L.dtype_code(inp.dtype), L.ptr(absmax), L.ptr(known_absmax), L.ptr(q_scale), L.stream_ptr())
        L.check(rc, "rmsnorm_forward")
        return
    x = inp.float()
    if inp2 is not None:
        x = (x + inp2.float()).to(inp.dtype)
        if residual_out is not None:
            residual_out.copy_(x)
        x = x.float()
    rs = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    n = (x * rs).to(inp.dtype)
    out = (n.float() * weight.float()).to(inp.dtype)
    if rstd is not None:
        rstd.copy_(rs.reshape(rstd.shape))
    if y is not None:
        y.copy_(out)
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, out.float().abs().max().reshape_as(absmax)))
    if q_out is not None:
        am = known_absmax.float().clamp_min(1e-10)
        q_out.copy_((out.float() * (448.0 / am)).clamp(-448, 448).to(q_out.dtype))
        if q_scale is not None:
            q_scale.copy_((am / 448.0).reshape_as(q_scale))


NORM_BWD_BLOCKS_PER_SM = 3         # persistent CTAs of the RMSNorm backward that share an SM


def rmsnorm_backward_scratch_elems(C: int, device) -> int:
    blocks = NORM_BWD_BLOCKS_PER_SM * num_sms(device) if torch.device(device).type == "cuda" else 1
    return blocks * C


def rmsnorm_backward(dinp: torch.Tensor, dweight: torch.Tensor, scratch: Optional[torch.Tensor], dout: torch.Tensor,
                     inp: torch.Tensor, weight: torch.Tensor, rstd: torch.Tensor, *, absmax: Optional[torch.Tensor] = None,
                     accumulate_dweight: bool = True) -> None:
    """dinp += d(rmsnorm)/d(inp) * dout;  dweight (+)= sum_rows dout * xhat."""
    C = inp.shape[-1]
    rows = inp.numel() // C
    if inp.is_cuda:
        blocks = NORM_BWD_BLOCKS_PER_SM * num_sms(inp.device)
        assert scratch is not None and scratch.numel() >= blocks * C and scratch.dtype == torch.float32
        rc = L.kernels().llmq_rmsnorm_backward(
            L.ptr(dinp), L.ptr(dweight), L.ptr(scratch), L.ptr(dout), L.ptr(inp), L.ptr(weight), L.ptr(rstd), rows, C,
            L.dtype_code(inp.dtype), L.ptr(absmax), int(accumulate_dweight), blocks, L.stream_ptr())
        L.check(rc, "rmsnorm_backward")
        return
    x = inp.float().reshape(rows, C)
    dy = dout.float().reshape(rows, C)
    rs = rstd.float().reshape(rows, 1)
    xh = x * rs
    w = weight.float()
    dot = (w * dy * xh).mean(-1, keepdim=True)
    g = (w * dy - xh * dot) * rs
    res = (dinp.float().reshape(rows, C) + g).to(dinp.dtype)
    dinp.copy_(res.reshape(dinp.shape))
    dw = (dy * xh).sum(0)
    if accumulate_dweight:
        dw = dw + dweight.float()
    dweight.copy_(dw.to(dweight.dtype))
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, dinp.float().abs().max().reshape_as(absmax)))


# =====================================================================================================
# SwiGLU
def swiglu_forward(out: Optional[torch.Tensor], inp: torch.Tensor, *, absmax: Optional[torch.Tensor] = None,
                   q_out: Optional[torch.Tensor] = None, known_absmax: Optional[torch.Tensor] = None,
                   q_scale: Optional[torch.Tensor] = None) -> None:
    """inp rows are [up | gate]; out = up * gate * sigmoid(gate)."""
    D = inp.shape[-1] // 2
    rows = inp.numel() // (2 * D)
    if inp.is_cuda:
        rc = L.kernels().llmq_swiglu_forward(L.ptr(out), L.ptr(q_out), L.ptr(inp), _ll(rows), D, L.dtype_code(inp.dtype),
                                             L.ptr(absmax), L.ptr(known_absmax), L.ptr(q_scale), num_sms(inp.device), L.stream_ptr())
        L.check(rc, "swiglu_forward")
        return
    x = inp.float().reshape(rows, 2 * D)
    up, gate = x[:, :D], x[:, D:]
    r = (up * gate * torch.sigmoid(gate)).to(inp.dtype)
    if out is not None:
        out.copy_(r.reshape(out.shape))
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, r.float().abs().max().reshape_as(absmax)))
    if q_out is not None:
        am = known_absmax.float().clamp_min(1e-10)
        q_out.copy_((r.float() * (448.0 / am)).clamp(-448, 448).to(q_out.dtype).reshape(q_out.shape))
        if q_scale is not None:
            q_scale.copy_((am / 448.0).reshape_as(q_scale))


def swiglu_forward_transposed(q_t: torch.Tensor, inp: torch.Tensor, *, known_absmax: torch.Tensor, q_scale: Optional[torch.Tensor] = None) -> None:
    """q_t[D, rows] (e4m3) = transpose of quantise(swiglu(inp[rows, 2D])) with an abs-max that is already known: the
    recompute path of an fp8 model whose weight-gradient GEMM reads the activation K-major.  Same bytes as
    ``swiglu_forward(q_out=...)`` followed by ``transpose``."""
    rows, D2 = inp.reshape(-1, inp.shape[-1]).shape
    D = D2 // 2
    if inp.is_cuda and inp.dtype == torch.bfloat16 and rows % 16 == 0 and D % 16 == 0:
        L.check(L.kernels().llmq_swiglu_forward_transposed(L.ptr(q_t), L.ptr(inp), rows, D, L.ptr(known_absmax), L.ptr(q_scale),
                                                           L.dtype_code(inp.dtype), L.stream_ptr()), "swiglu_forward_transposed")
        return
    tmp = torch.empty(rows, D, dtype=q_t.dtype, device=inp.device)
    swiglu_forward(None, inp.reshape(rows, D2), q_out=tmp, known_absmax=known_absmax, q_scale=q_scale)
    transpose(q_t, tmp)


def swiglu_backward(dinp: torch.Tensor, dout: torch.Tensor, inp: torch.Tensor, *, absmax: Optional[torch.Tensor] = None) -> None:
    """dinp = [d_up | d_gate]; may alias ``inp``."""
    D = inp.shape[-1] // 2
    rows = inp.numel() // (2 * D)
    if inp.is_cuda:
        rc = L.kernels().llmq_swiglu_backward(L.ptr(dinp), L.ptr(dout), L.ptr(inp), _ll(rows), D, L.dtype_code(inp.dtype),
                                              L.ptr(absmax), num_sms(inp.device), L.stream_ptr())
        L.check(rc, "swiglu_backward")
        return
    x = inp.float().reshape(rows, 2 * D)
    up, gate = x[:, :D], x[:, D:]
    d = dout.float().reshape(rows, D)
    s = torch.sigmoid(gate)
    du = d * gate * s
    dg = d * up * s * (1 + gate * (1 - s))
    r = torch.cat([du, dg], -1).to(dinp.dtype)
    dinp.copy_(r.reshape(dinp.shape))
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, r.float().abs().max().reshape_as(absmax)))


def swiglu_backward_stats(absmax: torch.Tensor, dout: torch.Tensor, inp: torch.Tensor, *, act_t: Optional[torch.Tensor] = None,
                          act_absmax: Optional[torch.Tensor] = None, act_scale: Optional[torch.Tensor] = None) -> None:
    """First pass of the SwiGLU backward of an fp8 model that never stores the 16-bit gradient: ``absmax`` is raised to the
    abs-max of [d_up | d_gate] (rounded to the activation type, as ``swiglu_backward`` would store it).  With ``act_t`` the
    same pass also writes ``act_t[D, rows]``, the transposed e4m3 SwiGLU output under the known ``act_absmax`` (what
    ``swiglu_forward_transposed`` computes), because it holds the up projection in registers anyway."""
    D = inp.shape[-1] // 2
    rows = inp.numel() // (2 * D)
    if inp.is_cuda and inp.dtype == torch.bfloat16 and rows % 16 == 0 and D % 16 == 0:
        L.check(L.kernels().llmq_swiglu_backward_stats(L.ptr(absmax), L.ptr(act_t), L.ptr(dout), L.ptr(inp), rows, D, L.ptr(act_absmax),
                                                       L.ptr(act_scale), L.dtype_code(inp.dtype), L.stream_ptr()), "swiglu_backward_stats")
        return
    tmp = torch.empty(rows, 2 * D, dtype=inp.dtype, device=inp.device)
    swiglu_backward(tmp, dout, inp, absmax=absmax)
    if act_t is not None:
        swiglu_forward_transposed(act_t, inp, known_absmax=act_absmax, q_scale=act_scale)


def swiglu_backward_quant(q_rows: torch.Tensor, q_t: torch.Tensor, scale_out: Optional[torch.Tensor], dout: torch.Tensor, inp: torch.Tensor,
                          absmax: torch.Tensor) -> None:
    """Second pass: ``q_rows[rows, 2D]`` = e4m3 copy of [d_up | d_gate] under ``absmax`` and ``q_t[2D, rows]`` its transpose; same
    bytes as ``swiglu_backward`` followed by ``quantize_transpose``."""
    D = inp.shape[-1] // 2
    rows = inp.numel() // (2 * D)
    if inp.is_cuda and inp.dtype == torch.bfloat16 and rows % 16 == 0 and D % 16 == 0 and q_rows.dtype == torch.float8_e4m3fn:
        L.check(L.kernels().llmq_swiglu_backward_quant(L.ptr(q_rows), L.ptr(q_t), L.ptr(scale_out), L.ptr(dout), L.ptr(inp), rows, D,
                                                       L.ptr(absmax), L.dtype_code(inp.dtype), L.stream_ptr()), "swiglu_backward_quant")
        return
    tmp = torch.empty(rows, 2 * D, dtype=inp.dtype, device=inp.device)
    swiglu_backward(tmp, dout, inp)
    quantize_transpose(q_rows, q_t, scale_out, tmp, absmax)


# =====================================================================================================
# RoPE
def rope_table(T: int, HS: int, theta: float, device) -> torch.Tensor:
    """(T, HS/2, 2) fp32 table of {cos, sin}."""
    device = torch.device(device)
    if device.type == "cuda":
        out = torch.empty(T, HS // 2, 2, dtype=torch.float32, device=device)
        with torch.cuda.device(device):
            L.check(L.kernels().llmq_rope_table(L.ptr(out), T, HS, _f(theta), L.stream_ptr()), "rope_table")
        return out
    d = torch.arange(HS // 2, dtype=torch.float64)
    inv = theta ** (-2.0 * d / HS)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
    return torch.stack([ang.cos(), ang.sin()], -1).float()


def rope(out: torch.Tensor, inp: torch.Tensor, freqs: torch.Tensor, Hq: int, Hkv: int, *, backward: bool = False,
         absmax: Optional[torch.Tensor] = None) -> None:
    """Rotates the q and k heads of packed (B, T, Hq+2Hkv, HS); ``out`` may be ``inp``."""
    B, T, H, HS = inp.shape
    assert H == Hq + 2 * Hkv
    if inp.is_cuda:
        rc = L.kernels().llmq_rope(L.ptr(out), L.ptr(inp), L.ptr(freqs), B, T, Hq, Hkv, HS, L.dtype_code(inp.dtype), int(backward),
                                   L.ptr(absmax), num_sms(inp.device), L.stream_ptr())
        L.check(rc, "rope")
        return
    x = inp.float()
    cos = freqs[:T, :, 0][None, :, None, :]
    sin = freqs[:T, :, 1][None, :, None, :]
    if backward:
        sin = -sin
    h = HS // 2
    x1, x2 = x[..., :h], x[..., h:]
    r1 = x1 * cos - x2 * sin
    r2 = x2 * cos + x1 * sin
    rot = torch.cat([r1, r2], -1)
    res = x.clone()
    res[:, :, :Hq + Hkv] = rot[:, :, :Hq + Hkv]
    res = res.to(out.dtype)
    out.copy_(res)
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, res.float().abs().max().reshape_as(absmax)))


# =====================================================================================================
# abs-max / quantisation / transposes / conversion / fill
def abs_max(out: torch.Tensor, x: torch.Tensor) -> None:
    """out = max(out, max|x|)  (``out`` is normally zeroed first)."""
    if x.is_cuda:
        L.check(L.kernels().llmq_abs_max(L.ptr(out), L.ptr(x), _ll(x.numel()), L.dtype_code(x.dtype), num_sms(x.device),
                                         L.stream_ptr()), "abs_max")
        return
    out.copy_(torch.maximum(out, x.float().abs().max().reshape_as(out)))


def quantize(out: torch.Tensor, scale_out: Optional[torch.Tensor], x: torch.Tensor, absmax: Optional[torch.Tensor]) -> None:
    """out = sat(x * QMAX / max(absmax, 1e-10)); scale_out = absmax / QMAX (1 when out is not an fp8 type)."""
    if x.is_cuda:
        L.check(L.kernels().llmq_quantize(L.ptr(out), L.ptr(scale_out), L.ptr(x), L.ptr(absmax), _ll(x.numel()), L.dtype_code(x.dtype),
                                          L.dtype_code(out.dtype), num_sms(x.device), L.stream_ptr()), "quantize")
        return
    if _is_f8(out.dtype):
        qm = _FP8_MAX[out.dtype]
        am = absmax.float().clamp_min(1e-10)
        out.copy_((x.float() * (qm / am)).clamp(-qm, qm).to(out.dtype).reshape(out.shape))
        if scale_out is not None:
            scale_out.copy_((am / qm).reshape_as(scale_out))
    else:
        out.copy_(x.to(out.dtype).reshape(out.shape))
        if scale_out is not None:
            scale_out.fill_(1.0)


def quantize_transpose(out_rows: Optional[torch.Tensor], out_t: torch.Tensor, scale_out: Optional[torch.Tensor], x: torch.Tensor,
                       absmax: Optional[torch.Tensor]) -> None:
    """One pass over ``x[rows, cols]``: ``out_rows`` (optional) = the fp8 copy, ``out_t[cols, rows]`` = its transpose.
    With a 1-byte ``x`` (and ``absmax`` None) the values are copied.  The transposed copy lets the weight-gradient GEMM
    read both operands K-major (reference: quantize_and_transpose_with_abs_max, src/kernels/quant.cu:100-193)."""
    x2 = x.reshape(-1, x.shape[-1])
    rows, cols = x2.shape
    if x.is_cuda and rows % 16 == 0 and cols % 16 == 0:
        L.check(L.kernels().llmq_quantize_transpose(L.ptr(out_rows), L.ptr(out_t), L.ptr(scale_out), L.ptr(x2), L.ptr(absmax), rows, cols,
                                                    L.dtype_code(x.dtype), L.dtype_code(out_t.dtype), L.stream_ptr()), "quantize_transpose")
        return
    if x2.element_size() == 1:
        if out_rows is not None:
            out_rows.reshape(rows, cols).copy_(x2)
        transpose(out_t, x2)
        return
    rows_q = out_rows.reshape(rows, cols) if out_rows is not None else torch.empty(rows, cols, dtype=out_t.dtype, device=x.device)
    quantize(rows_q, scale_out, x2, absmax)
    transpose(out_t, rows_q)


def transpose(out: torch.Tensor, x: torch.Tensor, *, absmax: Optional[torch.Tensor] = None,
              scale_out: Optional[torch.Tensor] = None) -> None:
    """out[c, r] = x[r, c]; with ``absmax`` the values are quantised to ``out.dtype`` on the way."""
    rows, cols = x.shape
    if x.is_cuda and out.element_size() == 1 and rows % 16 == 0 and cols % 16 == 0 and (absmax is not None or x.element_size() == 1):
        L.check(L.kernels().llmq_quantize_transpose(None, L.ptr(out), L.ptr(scale_out), L.ptr(x), L.ptr(absmax), rows, cols,
                                                    L.dtype_code(x.dtype), L.dtype_code(out.dtype), L.stream_ptr()), "transpose")
        return
    if x.is_cuda:
        L.check(L.kernels().llmq_transpose(L.ptr(out), L.ptr(scale_out), L.ptr(x), L.ptr(absmax), rows, cols, L.dtype_code(x.dtype),
                                           L.dtype_code(out.dtype), L.stream_ptr()), "transpose")
        return
    if absmax is not None:
        tmp = torch.empty(rows, cols, dtype=out.dtype)
        quantize(tmp, scale_out, x, absmax)
        out.copy_(tmp.view(torch.uint8).t().contiguous().view(out.dtype) if _is_f8(out.dtype) else tmp.t())
    else:
        out.copy_(x.view(torch.uint8).t().contiguous().view(x.dtype) if _is_f8(x.dtype) else x.t())


def convert(out: torch.Tensor, x: torch.Tensor) -> None:
    if x.is_cuda:
        L.check(L.kernels().llmq_convert(L.ptr(out), L.ptr(x), _ll(x.numel()), L.dtype_code(x.dtype), L.dtype_code(out.dtype),
                                         num_sms(x.device), L.stream_ptr()), "convert")
        return
    out.copy_(x.to(out.dtype).reshape(out.shape))


def fill(out: torch.Tensor, value: float) -> None:
    if out.is_cuda and out.dtype in (torch.bfloat16, torch.float32):
        L.check(L.kernels().llmq_fill(L.ptr(out), _f(value), _ll(out.numel()), L.dtype_code(out.dtype), num_sms(out.device),
                                      L.stream_ptr()), "fill")
        return
    out.fill_(value)


def fill_normal(out: torch.Tensor, mean: float, std: float, seed: int, subsequence: int = 0, offset: int = 0) -> None:
    """Counter-based N(mean, std): element i gets the value of counter ``offset + i`` of stream (seed, subsequence)."""
    if out.is_cuda:
        L.check(L.kernels().llmq_fill_normal(L.ptr(out), _ll(out.numel()), _f(mean), _f(std), ctypes.c_ulonglong(seed),
                                             ctypes.c_ulonglong(subsequence), _ll(offset), L.dtype_code(out.dtype),
                                             num_sms(out.device), L.stream_ptr()), "fill_normal")
        return
    # CPU: independent generator per (seed, subsequence); offset skips values so shards agree with the full tensor
    g = torch.Generator().manual_seed((seed * 1000003 + subsequence) % (2 ** 63))
    full = torch.randn(offset + out.numel(), generator=g, dtype=torch.float32)
    out.copy_((mean + std * full[offset:]).to(out.dtype).reshape(out.shape))


# =====================================================================================================
# Loss
def fused_classifier(logits: torch.Tensor, losses: torch.Tensor, lse: Optional[torch.Tensor], targets: torch.Tensor, dloss: float,
                     z_reg: float = 0.0, write_dlogits: bool = True) -> None:
    """Cross-entropy over rows of ``logits`` (rows, V): losses += lse - logit[target]; logits <- gradient in place."""
    rows, V = logits.shape
    if logits.is_cuda:
        L.check(L.kernels().llmq_fused_classifier(L.ptr(logits), L.ptr(losses), L.ptr(lse), L.ptr(targets), _f(dloss), _f(z_reg), rows, V,
                                                  _ll(logits.stride(0)), L.dtype_code(logits.dtype), int(write_dlogits),
                                                  L.stream_ptr()), "fused_classifier")
        return
    x = logits.float()
    tg = targets.reshape(rows).long()
    valid = (tg >= 0) & (tg < V)                # -100 and any other id outside the vocabulary: no loss, no gradient
    l = torch.logsumexp(x, -1)
    safe = tg.clamp(0, V - 1)
    picked = x.gather(1, safe[:, None])[:, 0]
    losses.reshape(rows).add_(torch.where(valid, l - picked, torch.zeros_like(l)))
    if lse is not None:
        lse.reshape(rows).copy_(torch.where(valid, l, torch.zeros_like(l)))
    if write_dlogits:
        p = torch.softmax(x, -1)
        g = p * (dloss + z_reg * l)[:, None]
        g[torch.arange(rows), safe] -= dloss
        g = torch.where(valid[:, None], g, torch.zeros_like(g))
        logits.copy_(g.to(logits.dtype))


def lse_stats(out: torch.Tensor, lse: torch.Tensor, accumulate: bool = False) -> None:
    """out = {max, sum} of the per-token log-sum-exp values."""
    if lse.is_cuda:
        L.check(L.kernels().llmq_lse_stats(L.ptr(out), L.ptr(lse), _ll(lse.numel()), int(accumulate), L.stream_ptr()), "lse_stats")
        return
    m, s = lse.float().max(), lse.float().sum()
    if accumulate:
        out[0] = torch.maximum(out[0], m)
        out[1] += s
    else:
        out[0], out[1] = m, s


def grouped_loss_sum(out: torch.Tensor, losses: torch.Tensor, group: int = 512) -> None:
    """out[g] = sum of losses(B, T) over the batch and positions [g*group, (g+1)*group)."""
    B, T = losses.shape
    if losses.is_cuda:
        L.check(L.kernels().llmq_grouped_loss_sum(L.ptr(out), L.ptr(losses), B, T, group, L.stream_ptr()), "grouped_loss_sum")
        return
    for g in range((T + group - 1) // group):
        out[g] = losses[:, g * group:(g + 1) * group].float().sum()


# =====================================================================================================
# Optimiser
def _sr_cpu(x: torch.Tensor, dtype: torch.dtype, gen: torch.Generator) -> torch.Tensor:
    if dtype == torch.float32:
        return x
    bits = x.contiguous().view(torch.int32)
    rnd = torch.randint(0, 1 << 16, bits.shape, generator=gen, dtype=torch.int32)
    return ((bits + rnd) & -65536).view(torch.float32).to(dtype)


def adamw(param: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, *, lr: float, beta1: float, beta2: float,
          step: int, eps: float, weight_decay: float, grad_scale: Optional[torch.Tensor] = None,
          absmax: Optional[torch.Tensor] = None, m_scales: Optional[torch.Tensor] = None, seed: int = 0,
          elem_offset: int = 0, stochastic: bool = True, hyper: Optional[torch.Tensor] = None) -> None:
    """In-place AdamW on flat shards; fp32 math, stochastic rounding when storing to bf16 / e4m3.

    ``hyper`` (GPU only, 8 fp32 values from ``adamw_hyper``): the step-dependent scalars are read from device memory, so
    the launch is the same every step (CUDA-graph replay); ``weight_decay`` then only selects (non-zero) or masks the decay
    and ``seed`` is an offset to the step's seed."""
    n = param.numel()
    if param.is_cuda:
        L.check(L.kernels().llmq_adamw_hyper(L.ptr(param), L.ptr(grad), L.ptr(m), L.ptr(v), L.ptr(m_scales), _ll(n), _f(lr), _f(beta1),
                                             _f(beta2), int(step), _f(eps), _f(weight_decay), L.ptr(grad_scale), L.ptr(absmax),
                                             ctypes.c_uint(seed & 0xFFFFFFFF), _ll(elem_offset), L.dtype_code(param.dtype),
                                             L.dtype_code(grad.dtype), L.dtype_code(m.dtype), L.dtype_code(v.dtype), num_sms(param.device),
                                             L.ptr(hyper), L.stream_ptr()), "adamw")
        return
    gen = torch.Generator().manual_seed((seed * 2654435761 + elem_offset) % (2 ** 63))
    g = grad.float().reshape(-1)
    if grad_scale is not None:
        g = g * grad_scale.float()
    p = param.float().reshape(-1)
    mf = m.float().reshape(-1)
    if _is_f8(m.dtype):
        mf = mf * m_scales.float().repeat_interleave(128)[:n]
    vf = v.float().reshape(-1)
    mf = beta1 * mf + (1 - beta1) * g
    vf = beta2 * vf + (1 - beta2) * g * g
    mh = mf / (1 - beta1 ** step)
    vh = vf / (1 - beta2 ** step)
    p = p - lr * (mh / (vh.sqrt() + eps) + weight_decay * p)
    rnd = (lambda x, dt: _sr_cpu(x, dt, gen)) if stochastic else (lambda x, dt: x.to(dt))
    param.copy_(rnd(p, param.dtype).reshape(param.shape))
    v.copy_(rnd(vf, v.dtype).reshape(v.shape))
    if _is_f8(m.dtype):
        blocks = mf.reshape(-1, 128)
        sc = blocks.abs().amax(-1).clamp_min(1e-30) / 448.0
        m.copy_((blocks / sc[:, None]).clamp(-448, 448).to(m.dtype).reshape(m.shape))
        m_scales.copy_(sc.reshape(m_scales.shape))
    else:
        m.copy_(rnd(mf, m.dtype).reshape(m.shape))
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, param.float().abs().max().reshape_as(absmax)))


def adamw_hyper(out: torch.Tensor, *, lr: float, beta1: float, beta2: float, step: int, eps: float, weight_decay: float, seed: int) -> None:
    """Fills the 8 fp32 values that ``adamw(..., hyper=...)`` reads (``out``: pinned host tensor), with the arithmetic of
    the by-value launch (fp32 bias corrections)."""
    L.kernels().llmq_adamw_fill_hyper(L.ptr(out), _f(lr), _f(beta1), _f(beta2), int(step), _f(eps), _f(weight_decay),
                                      ctypes.c_uint(seed & 0xFFFFFFFF))


NORM_PARTIALS = 512


def norm_squared(partials: torch.Tensor, x: torch.Tensor) -> None:
    """partials[b] += partial sum of squares of x (deterministic per-block slots)."""
    if x.is_cuda:
        L.check(L.kernels().llmq_norm_squared(L.ptr(partials), L.ptr(x), _ll(x.numel()), L.dtype_code(x.dtype), partials.numel(),
                                              L.stream_ptr()), "norm_squared")
        return
    partials[0] += x.float().pow(2).sum()


def deterministic_sum(out: torch.Tensor, x: torch.Tensor) -> None:
    if x.is_cuda:
        L.check(L.kernels().llmq_deterministic_sum(L.ptr(out), L.ptr(x), x.numel(), L.stream_ptr()), "deterministic_sum")
        return
    out.copy_(x.float().sum().reshape_as(out))


def norm_finish(io: torch.Tensor, clip: float, host_norm: Optional[torch.Tensor] = None) -> None:
    """io[0]: squared norm -> norm; io[1] <- clip multiplier (min(1, clip / norm); 0 for a non-finite norm)."""
    if io.is_cuda:
        L.check(L.kernels().llmq_norm_finish(L.ptr(io), _f(clip), L.ptr(host_norm), L.stream_ptr()), "norm_finish")
        return
    norm = io[0].sqrt()
    scale = torch.ones(())
    if clip > 0 and norm > clip:
        scale = clip / norm
    if not torch.isfinite(norm):
        scale = torch.zeros(())
    io[0] = norm
    io[1] = scale
    if host_norm is not None:
        host_norm.copy_(norm.reshape_as(host_norm))


def vector_add_sr(dst: torch.Tensor, a: torch.Tensor, b: torch.Tensor, scale: float = 1.0, seed: int = 0) -> None:
    """dst = SR(scale * (a + b))."""
    if dst.is_cuda:
        L.check(L.kernels().llmq_vector_add_sr(L.ptr(dst), L.ptr(a), L.ptr(b), _f(scale), _ll(dst.numel()), ctypes.c_uint(seed & 0xFFFFFFFF),
                                               L.dtype_code(dst.dtype), num_sms(dst.device), L.stream_ptr()), "vector_add_sr")
        return
    gen = torch.Generator().manual_seed(seed)
    r = scale * (a.float() + b.float())
    dst.copy_(_sr_cpu(r.reshape(-1), dst.dtype, gen).reshape(dst.shape))


def vector_reduce_sr(dst: torch.Tensor, src: torch.Tensor, scale: float, n_shards: int, *, skip: int = -1,
                     accumulate: bool = False, seed: int = 0) -> None:
    """dst = SR(scale * (sum_{k != skip} src[k] (+ dst))), src is (n_shards, dst.numel())."""
    n = dst.numel()
    if dst.is_cuda:
        L.check(L.kernels().llmq_vector_reduce_sr(L.ptr(dst), L.ptr(src), _f(scale), n_shards, skip, _ll(n), int(accumulate), _ll(n),
                                                  ctypes.c_uint(seed & 0xFFFFFFFF), L.dtype_code(dst.dtype), num_sms(dst.device),
                                                  L.stream_ptr()), "vector_reduce_sr")
        return
    gen = torch.Generator().manual_seed(seed)
    s = src.float().reshape(n_shards, n)
    acc = dst.float().reshape(-1).clone() if accumulate else torch.zeros(n)
    for k in range(n_shards):
        if k != skip:
            acc = acc + s[k]
    dst.copy_(_sr_cpu(acc * scale, dst.dtype, gen).reshape(dst.shape))


# =====================================================================================================
# Embedding / bias
def encoder_forward(out: torch.Tensor, tokens: torch.Tensor, wte: torch.Tensor) -> None:
    V, C = wte.shape
    if out.is_cuda:
        L.check(L.kernels().llmq_encoder_forward(L.ptr(out), L.ptr(tokens), L.ptr(wte), _ll(tokens.numel()), C, V, L.dtype_code(wte.dtype),
                                                 num_sms(out.device), L.stream_ptr()), "encoder_forward")
        return
    out.copy_(wte[tokens.reshape(-1).long().clamp(0, V - 1)].reshape(out.shape))


def encoder_backward(dwte: torch.Tensor, dout: torch.Tensor, tokens: torch.Tensor) -> None:
    """dwte[tok] += sum of dout rows with that token; deterministic (positions are summed in ascending order).
    On the GPU everything happens in kernels on the current stream (no sort, no host synchronisation); token ids outside
    the vocabulary are skipped."""
    V, C = dwte.shape
    flat = tokens.reshape(-1)
    if dwte.is_cuda:
        BT = flat.numel()
        scratch = _scratch("encoder_bwd_rank", dwte.device, (2 * BT,), torch.int32)
        L.check(L.kernels().llmq_encoder_backward(L.ptr(dwte), L.ptr(dout), L.ptr(flat), L.ptr(scratch), BT, C, V,
                                                  L.dtype_code(dwte.dtype), L.stream_ptr()), "encoder_backward")
        return
    ok = (flat >= 0) & (flat < V)
    acc = dwte.float()
    acc.index_add_(0, flat[ok].long(), dout.float().reshape(-1, C)[ok])
    dwte.copy_(acc.to(dwte.dtype))


def bias_backward(dbias: torch.Tensor, dout: torch.Tensor, scratch: Optional[torch.Tensor], *, scale_a: Optional[torch.Tensor] = None,
                  scale_b: Optional[torch.Tensor] = None, accumulate: bool = True) -> None:
    """dbias (+)= scale * sum_rows dout (dout may be fp8 with a dequantisation factor)."""
    C = dout.shape[-1]
    rows = dout.numel() // C
    if dout.is_cuda:
        slices = 64
        assert scratch is not None and scratch.numel() >= slices * C
        L.check(L.kernels().llmq_bias_backward(L.ptr(dbias), L.ptr(scratch), L.ptr(dout), _ll(rows), C, slices, L.ptr(scale_a), L.ptr(scale_b),
                                               int(accumulate), L.dtype_code(dout.dtype), L.dtype_code(dbias.dtype), L.stream_ptr()),
                "bias_backward")
        return
    s = dout.float().reshape(rows, C).sum(0)
    if scale_a is not None:
        s = s * scale_a.float()
    if scale_b is not None:
        s = s * scale_b.float()
    if accumulate:
        s = s + dbias.float()
    dbias.copy_(s.to(dbias.dtype))


# =====================================================================================================
# Attention
def attention_forward(out: torch.Tensor, lse: torch.Tensor, qkv: torch.Tensor, Hq: int, Hkv: int,
                      absmax: Optional[torch.Tensor] = None) -> None:
    """Causal GQA attention on packed qkv (B,T,Hq+2Hkv,HS): out (B,T,Hq,HS), lse (B,Hq,T) natural log.
    ``absmax`` (optional) is raised to max |out|."""
    B, T, H, HS = qkv.shape
    if qkv.is_cuda and qkv.dtype == torch.float32:
        # fp32 model: the tensor-core kernel works on bf16 copies (fp32 softmax statistics and accumulation inside)
        qh, oh = _attn_half("qkv", qkv), _attn_half("out", out)
        convert(qh, qkv)
        attention_forward(oh, lse, qh, Hq, Hkv)
        convert(out, oh)
        if absmax is not None:
            abs_max(absmax, out)
        return
    if qkv.is_cuda:
        assert qkv.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
        L.check(L.kernels().llmq_attention_forward(L.ptr(out), L.ptr(lse), L.ptr(qkv), B, T, Hq, Hkv, HS, L.ptr(absmax),
                                                   L.ptr(status_word(qkv.device)), L.stream_ptr()), "attention_forward")
        return
    o, l = _attention_ref(qkv.float(), Hq, Hkv)
    out.copy_(o.to(out.dtype))
    lse.copy_(l)
    if absmax is not None:
        absmax.copy_(torch.maximum(absmax, out.float().abs().max().reshape_as(absmax)))


def _attn_half(tag: str, like: torch.Tensor) -> torch.Tensor:
    """bf16 scratch of the shape of ``like``."""
    return _scratch("attn_" + tag, like.device, like.shape, torch.bfloat16)


def _attention_ref(qkv: torch.Tensor, Hq: int, Hkv: int):
    B, T, H, HS = qkv.shape
    q = qkv[:, :, :Hq].permute(0, 2, 1, 3)
    k = qkv[:, :, Hq:Hq + Hkv].permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    v = qkv[:, :, Hq + Hkv:].permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, 1)
    s = (q @ k.transpose(-1, -2)) / math.sqrt(HS)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    s = s.masked_fill(~mask, float("-inf"))
    l = torch.logsumexp(s, -1)
    p = torch.exp(s - l[..., None])
    o = (p @ v).permute(0, 2, 1, 3)
    return o, l


def attention_backward(dqkv: torch.Tensor, scratch: Optional[torch.Tensor], dout: torch.Tensor, out: torch.Tensor, lse: torch.Tensor,
                       qkv: torch.Tensor, Hq: int, Hkv: int) -> None:
    """Packed gradient of :func:`attention_forward`; ``scratch`` holds B*Hq*T floats."""
    B, T, H, HS = qkv.shape
    if qkv.is_cuda and qkv.dtype == torch.float32:
        qh, oh, dh, gh = _attn_half("qkv", qkv), _attn_half("out", out), _attn_half("dout", dout), _attn_half("dqkv", dqkv)
        convert(qh, qkv)
        convert(oh, out)
        convert(dh, dout)
        attention_backward(gh, scratch, dh, oh, lse, qh, Hq, Hkv)
        convert(dqkv, gh)
        return
    if qkv.is_cuda:
        assert qkv.dtype == torch.bfloat16 and dqkv.dtype == torch.bfloat16
        assert scratch is not None and scratch.numel() >= B * Hq * T
        L.check(L.kernels().llmq_attention_backward(L.ptr(dqkv), L.ptr(scratch), L.ptr(dout), L.ptr(out), L.ptr(lse), L.ptr(qkv), B, T, Hq, Hkv,
                                                    HS, L.ptr(status_word(qkv.device)), L.stream_ptr()), "attention_backward")
        return
    # written out (no autograd): this also runs below the autograd dispatch key, inside a torch custom op
    x, G = qkv.float(), Hq // Hkv
    q = x[:, :, :Hq].permute(0, 2, 1, 3)
    k = x[:, :, Hq:Hq + Hkv].permute(0, 2, 1, 3).repeat_interleave(G, 1)
    v = x[:, :, Hq + Hkv:].permute(0, 2, 1, 3).repeat_interleave(G, 1)
    scale = 1.0 / math.sqrt(HS)
    mask = torch.ones(T, T, dtype=torch.bool, device=qkv.device).tril()
    p = torch.softmax(((q @ k.transpose(-1, -2)) * scale).masked_fill(~mask, float("-inf")), -1)
    do = dout.float().permute(0, 2, 1, 3)
    dv = p.transpose(-1, -2) @ do
    dp = do @ v.transpose(-1, -2)
    ds = p * (dp - (dp * p).sum(-1, keepdim=True)) * scale
    dq = ds @ k
    dk = ds.transpose(-1, -2) @ q
    dk = dk.reshape(B, Hkv, G, T, HS).sum(2)
    dv = dv.reshape(B, Hkv, G, T, HS).sum(2)
    g = torch.cat([dq.permute(0, 2, 1, 3), dk.permute(0, 2, 1, 3), dv.permute(0, 2, 1, 3)], 2)
    dqkv.copy_(g.to(dqkv.dtype))


# =====================================================================================================
# QK-norm (kernel API parity; not used by the Llama / Qwen2 training path)
def qk_norm_forward(out: torch.Tensor, rstd: torch.Tensor, qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor,
                    eps: float, Hq: int, Hkv: int) -> None:
    """Per-head RMSNorm of the q and k heads of packed (B,T,Hq+2Hkv,HS); v heads of ``out`` are left as they are
    (pass ``out = qkv`` for the in-place form).  rstd: (B*T, Hq+Hkv)."""
    B, T, H, HS = qkv.shape
    if qkv.is_cuda:
        L.check(L.kernels().llmq_qk_norm_forward(L.ptr(out), L.ptr(rstd), L.ptr(qkv), L.ptr(q_weight), L.ptr(k_weight), _f(eps), _ll(B * T),
                                                 Hq, Hkv, HS, L.dtype_code(qkv.dtype), L.stream_ptr()), "qk_norm_forward")
        return
    x = qkv.float()[:, :, :Hq + Hkv]
    rs = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    w = torch.cat([q_weight.float().expand(Hq, HS), k_weight.float().expand(Hkv, HS)], 0)
    y = ((x * rs).to(qkv.dtype).float() * w).to(out.dtype)
    out[:, :, :Hq + Hkv] = y
    rstd.copy_(rs.reshape(rstd.shape))


def qk_norm_backward(dqkv: torch.Tensor, dq_weight: torch.Tensor, dk_weight: torch.Tensor, scratch: Optional[torch.Tensor], dout: torch.Tensor,
                     qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, rstd: torch.Tensor, Hq: int, Hkv: int,
                     accumulate: bool = False) -> None:
    """Gradient of :func:`qk_norm_forward` for the q and k heads (v heads of ``dqkv`` untouched); scratch: 128*2*HS floats."""
    B, T, H, HS = qkv.shape
    if qkv.is_cuda:
        slices = 128
        assert scratch is not None and scratch.numel() >= slices * 2 * HS
        L.check(L.kernels().llmq_qk_norm_backward(L.ptr(dqkv), L.ptr(dq_weight), L.ptr(dk_weight), L.ptr(scratch), L.ptr(dout), L.ptr(qkv),
                                                  L.ptr(q_weight), L.ptr(k_weight), L.ptr(rstd), _ll(B * T), Hq, Hkv, HS, slices,
                                                  int(accumulate), L.dtype_code(qkv.dtype), L.stream_ptr()), "qk_norm_backward")
        return
    HN = Hq + Hkv
    x = qkv.float()[:, :, :HN]
    dy = dout.float()[:, :, :HN]
    rs = rstd.float().reshape(B, T, HN, 1)
    w = torch.cat([q_weight.float().expand(Hq, HS), k_weight.float().expand(Hkv, HS)], 0)
    xh = x * rs
    dot = (w * dy * xh).mean(-1, keepdim=True)
    dqkv[:, :, :HN] = ((w * dy - xh * dot) * rs).to(dqkv.dtype)
    dwq = (dy[:, :, :Hq] * xh[:, :, :Hq]).sum((0, 1, 2))
    dwk = (dy[:, :, Hq:] * xh[:, :, Hq:]).sum((0, 1, 2))
    if accumulate:
        dwq, dwk = dwq + dq_weight.float(), dwk + dk_weight.float()
    dq_weight.copy_(dwq.to(dq_weight.dtype))
    dk_weight.copy_(dwk.to(dk_weight.dtype))
