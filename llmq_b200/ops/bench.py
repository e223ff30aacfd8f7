"""Kernel micro-benchmarks: device-timed (CUDA events), warmed up, L2 flushed between iterations.

    python -m llmq_b200.ops.bench gemm --m 16384 --n 37888 --k 3584 --dtype fp8 [--a-mn] [--b-mn] [--mode 0|1|2]
    python -m llmq_b200.ops.bench attention --b 8 --t 2048 --hq 28 --hkv 4 --hs 128
    python -m llmq_b200.ops.bench elementwise --rows 16384 --c 3584 --d 18944
    python -m llmq_b200.ops.bench adamw --numel 134217728

Prints achieved TFLOP/s or GB/s and, when ``MEASURED_PEAKS.json`` is found at the repository root, the
fraction of the measured cuBLAS bf16 / copy-bandwidth peak.  ``--iters 1 --no-flush`` gives a run that is
convenient to capture under a profiler.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from . import kernels as K
from . import lib as L

DEV = "cuda"


def _peaks():
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return d.get("bf16_tflops", 1590.0), d.get("hbm_gbs", 6650.0), "measured"
    return 1590.0, 6650.0, "fallback"


class Timer:
    def __init__(self, iters, warmup, flush):
        self.iters, self.warmup = iters, warmup
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV) if flush else None

    def time(self, fn):
        for _ in range(self.warmup):
            fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(self.iters):
            if self.flush is not None:
                self.flush.zero_()                      # evicts the 126 MB L2
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        K.check_status(torch.device(DEV, torch.cuda.current_device()))
        return total / self.iters


def _rand(shape, dtype):
    t = torch.randn(*shape, device=DEV)
    return t.to(dtype)


def bench_gemm(a, tm):
    dt = {"bf16": torch.bfloat16, "fp8": torch.float8_e4m3fn, "e4m3": torch.float8_e4m3fn, "fp32": torch.float32}[a.dtype]
    L.kernels().llmq_gemm_set_mode(a.mode)
    A = _rand((a.k, a.m) if a.a_mn else (a.m, a.k), dt)
    B = _rand((a.k, a.n) if a.b_mn else (a.n, a.k), dt)
    C = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=DEV)
    bias = _rand((a.n,), torch.bfloat16) if a.bias else None
    ms = tm.time(lambda: K.gemm(C, A, B, a_mn=a.a_mn, b_mn=a.b_mn, accumulate=a.accumulate, bias=bias))
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    peak, _, src = _peaks()
    print(json.dumps({"op": "gemm", "m": a.m, "n": a.n, "k": a.k, "dtype": a.dtype, "a_mn": a.a_mn, "b_mn": a.b_mn, "bias": a.bias, "mode": a.mode,
                      "ms": round(ms, 4), "tflops": round(tf, 1), f"frac_of_{src}_bf16_peak": round(tf / peak, 3)}))


def bench_gemm_mx(a, tm):
    """Block-scaled e4m3 GEMM and its two quantisers (along rows / along columns with transpose)."""
    x = _rand((a.m, a.k), torch.bfloat16)
    w = _rand((a.n, a.k), torch.bfloat16)
    aq, asf = K.quantize_mx(x, operand="a")
    bq, bsf = K.quantize_mx(w, operand="b")
    C = torch.empty(a.m, a.n, dtype=torch.bfloat16, device=DEV)
    ms = tm.time(lambda: K.gemm_mx(C, aq, asf, bq, bsf, accumulate=a.accumulate))
    tf = 2.0 * a.m * a.n * a.k / ms / 1e9
    peak, bw, src = _peaks()
    out = {"op": "gemm_mx", "m": a.m, "n": a.n, "k": a.k, "ms": round(ms, 4), "tflops": round(tf, 1), f"frac_of_{src}_bf16_peak": round(tf / peak, 3)}
    nbytes = a.m * a.k * 3 + a.m * a.k // 32
    ms_q = tm.time(lambda: K.quantize_mx(x, operand="a", q_out=aq, sf_out=asf))
    out["quantize_rows_ms"] = round(ms_q, 4); out[f"quantize_rows_frac_of_{src}_bw"] = round(nbytes / ms_q / 1e6 / bw, 3)
    if a.m % 128 == 0:
        tq, tsf = K.quantize_mx(x, transpose=True, operand="b")
        ms_t = tm.time(lambda: K.quantize_mx(x, transpose=True, operand="b", q_out=tq, sf_out=tsf))
        out["quantize_cols_ms"] = round(ms_t, 4); out[f"quantize_cols_frac_of_{src}_bw"] = round(nbytes / ms_t / 1e6 / bw, 3)
        if a.k % 128 == 0:
            bufs = K.quantize_mx_both(x)
            ms_b = tm.time(lambda: K.quantize_mx_both(x, q_rows=bufs[0], sf_rows=bufs[1], q_cols=bufs[2], sf_cols=bufs[3]))
            out["quantize_both_ms"] = round(ms_b, 4)
            out[f"quantize_both_frac_of_{src}_bw"] = round((a.m * a.k * 4 + a.m * a.k // 16) / ms_b / 1e6 / bw, 3)
    print(json.dumps(out))


def bench_attention(a, tm):
    qkv = _rand((a.b, a.t, a.hq + 2 * a.hkv, a.hs), torch.bfloat16)
    out = torch.empty(a.b, a.t, a.hq, a.hs, dtype=torch.bfloat16, device=DEV)
    lse = torch.empty(a.b, a.hq, a.t, device=DEV)
    dout = _rand((a.b, a.t, a.hq, a.hs), torch.bfloat16)
    dqkv = torch.empty_like(qkv)
    scratch = torch.empty(a.b * a.hq * a.t, device=DEV)
    fwd = tm.time(lambda: K.attention_forward(out, lse, qkv, a.hq, a.hkv))
    bwd = tm.time(lambda: K.attention_backward(dqkv, scratch, dout, out, lse, qkv, a.hq, a.hkv))
    flops_fwd = 4.0 * a.b * a.hq * a.t * a.t * a.hs / 2          # causal: half of the score matrix
    peak, _, src = _peaks()
    print(json.dumps({"op": "attention", "b": a.b, "t": a.t, "hq": a.hq, "hkv": a.hkv, "hs": a.hs,
                      "fwd_ms": round(fwd, 4), "fwd_tflops": round(flops_fwd / fwd / 1e9, 1),
                      "bwd_ms": round(bwd, 4), "bwd_tflops": round(2.5 * flops_fwd / bwd / 1e9, 1),
                      f"fwd_frac_of_{src}_bf16_peak": round(flops_fwd / fwd / 1e9 / peak, 3)}))


def bench_elementwise(a, tm):
    _, bw, src = _peaks()
    rows, C, D = a.rows, a.c, a.d
    res = {}
    x, y, w = _rand((rows, C), torch.bfloat16), _rand((rows, C), torch.bfloat16), _rand((C,), torch.bfloat16)
    o, r = torch.empty_like(x), torch.empty_like(x)
    rstd, am = torch.empty(rows, device=DEV), torch.zeros(1, device=DEV)
    ms = tm.time(lambda: K.rmsnorm_forward(o, rstd, x, w, 1e-6, residual_out=r, inp2=y, absmax=am))
    res["fused_residual_rmsnorm"] = (ms, 4 * rows * C * 2)
    scratch = torch.empty(K.rmsnorm_backward_scratch_elems(C, DEV), device=DEV)
    dw = torch.zeros(C, dtype=torch.bfloat16, device=DEV)
    ms = tm.time(lambda: K.rmsnorm_backward(o, dw, scratch, y, x, w, rstd, absmax=am))
    res["rmsnorm_backward"] = (ms, 4 * rows * C * 2)
    q = torch.empty(rows, C, dtype=torch.float8_e4m3fn, device=DEV)
    sc = torch.empty(1, device=DEV)
    am.fill_(4.0)
    ms = tm.time(lambda: K.quantize(q, sc, x, am))
    res["quantize_e4m3"] = (ms, rows * C * 3)
    up, sw = _rand((rows, 2 * D), torch.bfloat16), torch.empty(rows, D, dtype=torch.bfloat16, device=DEV)
    ms = tm.time(lambda: K.swiglu_forward(sw, up, absmax=am))
    res["swiglu_forward"] = (ms, rows * D * 6)
    # the fp8 K-major backward path: what it replaced (bf16 gradient, then quantise + transpose, plus the transposed recompute)
    # and its two passes
    F8 = torch.float8_e4m3fn
    dq, dqt, act_t = torch.empty(rows, 2 * D, dtype=F8, device=DEV), torch.empty(2 * D, rows, dtype=F8, device=DEV), torch.empty(D, rows, dtype=F8, device=DEV)
    dgrad = torch.empty(rows, 2 * D, dtype=torch.bfloat16, device=DEV)
    am2, sc2 = torch.full((1,), 8.0, device=DEV), torch.empty(1, device=DEV)
    ms = tm.time(lambda: K.swiglu_backward(dgrad, sw, up, absmax=am))
    res["swiglu_backward_out_of_place"] = (ms, rows * D * 10)
    ms = tm.time(lambda: K.quantize_transpose(dq, dqt, sc, dgrad, am))
    res["quantize_transpose_dup"] = (ms, rows * D * 8)
    ms = tm.time(lambda: K.swiglu_forward_transposed(act_t, up, known_absmax=am2, q_scale=sc2))
    res["swiglu_forward_transposed"] = (ms, rows * D * 5)
    ms = tm.time(lambda: K.swiglu_backward_stats(am, sw, up))
    res["swiglu_backward_stats"] = (ms, rows * D * 6)
    ms = tm.time(lambda: K.swiglu_backward_stats(am, sw, up, act_t=act_t, act_absmax=am2, act_scale=sc2))
    res["swiglu_backward_stats_with_act"] = (ms, rows * D * 7)
    ms = tm.time(lambda: K.swiglu_backward_quant(dq, dqt, sc, sw, up, am))
    res["swiglu_backward_quant"] = (ms, rows * D * 10)
    del dq, dqt, act_t, dgrad
    ms = tm.time(lambda: K.swiglu_backward(up, sw, up, absmax=am))
    res["swiglu_backward"] = (ms, rows * D * 10)
    swq = torch.empty(rows, D, dtype=torch.float8_e4m3fn, device=DEV)
    up2 = _rand((rows, 2 * D), torch.bfloat16)
    am.fill_(8.0)
    ms = tm.time(lambda: K.swiglu_forward(None, up2, q_out=swq, known_absmax=am, q_scale=sc))
    res["swiglu_forward_quant"] = (ms, rows * D * 5)
    ms = tm.time(lambda: K.quantize(swq, sc, sw, am))
    res["quantize_e4m3_large"] = (ms, rows * D * 3)
    ms = tm.time(lambda: K.abs_max(am, x))
    res["abs_max"] = (ms, rows * C * 2)
    hq, hkv, hs = 28, 4, 128
    qkv = _rand((rows // 2048, 2048, hq + 2 * hkv, hs), torch.bfloat16)
    freqs = K.rope_table(2048, hs, 1e6, DEV)
    ms = tm.time(lambda: K.rope(qkv, qkv, freqs, hq, hkv, absmax=am))
    res["rope"] = (ms, qkv.numel() * 4)
    out = {k: {"ms": round(v[0], 4), "gbs": round(v[1] / v[0] / 1e6, 1), f"frac_of_{src}_hbm": round(v[1] / v[0] / 1e6 / bw, 3)} for k, v in res.items()}
    print(json.dumps({"op": "elementwise", "rows": rows, "c": C, "d": D, **out}))


def bench_adamw(a, tm):
    _, bw, src = _peaks()
    n = a.numel
    p, g = _rand((n,), torch.bfloat16), _rand((n,), torch.bfloat16)
    m, v = torch.zeros(n, dtype=torch.bfloat16, device=DEV), torch.zeros(n, dtype=torch.bfloat16, device=DEV)
    gs, am = torch.ones(1, device=DEV), torch.zeros(1, device=DEV)
    ms = tm.time(lambda: K.adamw(p, g, m, v, lr=1e-4, beta1=0.9, beta2=0.95, step=3, eps=1e-8, weight_decay=0.1, grad_scale=gs, absmax=am, seed=1))
    gbs = n * 14 / ms / 1e6
    print(json.dumps({"op": "adamw_bf16", "n": n, "ms": round(ms, 4), "gbs": round(gbs, 1), f"frac_of_{src}_hbm": round(gbs / bw, 3)}))


def bench_p2p(a, tm):
    """The peer-memory collective kernels with every "rank" living on this one GPU: the peer table holds local buffers,
    so the kernels run exactly as on several GPUs but all traffic stays in local HBM (what the numbers show is the
    kernels' own efficiency, not NVLink)."""
    import ctypes
    _, bw, src = _peaks()
    w = a.world
    rows, cols = a.rows, a.c
    n_shard = rows * cols // w
    shard = _rand((n_shard,), torch.bfloat16)
    gathers = [torch.empty(rows * cols, dtype=torch.float8_e4m3fn, device=DEV) for _ in range(w)]
    peers = (ctypes.c_void_p * 8)(*([g.data_ptr() for g in gathers] + [0] * (8 - w)))
    am, sc = torch.full((1,), 4.0, device=DEV), torch.zeros(1, device=DEV)
    sms = K.num_sms(torch.device(DEV, torch.cuda.current_device()))
    k = L.kernels()
    res = {}
    ms = tm.time(lambda: L.check(k.llmq_p2p_quant_allgather(peers, ctypes.c_longlong(0), L.ptr(shard), ctypes.c_longlong(n_shard), 0, w, L.ptr(am),
                                                             L.ptr(sc), 1, sms, L.stream_ptr()), "p2p_quant_allgather"))
    res["quant_allgather_e4m3"] = (ms, n_shard * (2 + w))              # read bf16 shard, write one e4m3 copy per rank
    grads = [_rand((rows * cols,), torch.bfloat16) for _ in range(w)]
    gpeers = (ctypes.c_void_p * 8)(*([g.data_ptr() for g in grads] + [0] * (8 - w)))
    dst = torch.zeros(n_shard, dtype=torch.bfloat16, device=DEV)
    parts = torch.zeros(K.NORM_PARTIALS, device=DEV)
    ms = tm.time(lambda: L.check(k.llmq_p2p_reduce_scatter(gpeers, None, ctypes.c_longlong(0), ctypes.c_longlong(n_shard), 0, w, L.ptr(dst), 1,
                                                            ctypes.c_float(1.0 / w), L.ptr(parts), K.NORM_PARTIALS, ctypes.c_uint(7), sms,
                                                            L.stream_ptr()), "p2p_reduce_scatter"))
    res["reduce_scatter_sr_norm"] = (ms, n_shard * 2 * (w + 2))          # read one slice per rank + old shard, write shard
    out = {kk: {"ms": round(v[0], 4), "gbs": round(v[1] / v[0] / 1e6, 1), f"frac_of_{src}_hbm": round(v[1] / v[0] / 1e6 / bw, 3)} for kk, v in res.items()}
    print(json.dumps({"op": "p2p_single_gpu_emulation", "world": w, "elements": rows * cols, **out}))


def bench_fused_gemm(a, tm):
    """The two GEMMs that carry a collective, with every "rank" on this one GPU (rank 0 runs, the peer tables point at
    local buffers, the peers' arrivals are booked in advance), against the plain GEMM of the same shape:

    * GEMM -> reduce-scatter (weight gradient, both operands MN-major): the epilogue stores every row block into its
      owner's landing buffer and bumps the owner's counter; the tail sums this rank's slots into the shard.
    * all-gather -> GEMM (first consumer of gathered weights): the TMA producer polls one arrival flag per source
      rank before it loads that rank's rows of B.

    What the numbers show is what the collective part costs inside the kernel; no byte crosses NVLink here."""
    import ctypes
    dev = torch.device(DEV, torch.cuda.current_device())
    st = K._dev_state(dev)
    k = L.kernels()
    w = a.world
    peak, _, src = _peaks()
    f8 = torch.float8_e4m3fn
    out = {"op": "fused_gemm_single_gpu_emulation", "world": w}
    # ---- dW = dY^T @ X, reduce-scattered over rows
    M, N, Kd = a.m, a.n, a.k
    At, Bt = _rand((Kd, M), f8), _rand((Kd, N), f8)
    ones = torch.ones(1, device=DEV)
    plain = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    ms_plain = tm.time(lambda: K.gemm(plain, At, Bt, a_mn=True, b_mn=True, scale_a=ones, scale_b=ones))
    landing = [torch.zeros(w, M // w, N, dtype=torch.bfloat16, device=DEV) for _ in range(w)]
    counters = torch.zeros(w, 64, dtype=torch.int32, device=DEV)               # one counter per "rank", 256 bytes apart
    shard = torch.zeros(M // w, N, dtype=torch.bfloat16, device=DEV)
    parts = torch.zeros(K.NORM_PARTIALS, device=DEV)
    land_arr = (ctypes.c_void_p * 8)(*([t.data_ptr() for t in landing] + [0] * (8 - w)))
    cnt_arr = (ctypes.c_void_p * 8)(*([counters[i].data_ptr() for i in range(w)] + [0] * (8 - w)))
    arrivals = int(k.llmq_gemm_rs_arrivals(M, N, w))
    state = {"target": 0}

    def run_rs():
        # the other ranks' share of the arrivals at rank 0 is booked before the launch
        state["target"] += arrivals
        counters[0, 0] += arrivals - arrivals // w
        L.check(k.llmq_gemm_rs(L.ptr(At), L.ptr(Bt), L.ptr(landing[0]), M, N, Kd, 1, 1, 1, 1, ctypes.c_longlong(M), ctypes.c_longlong(N), 0,
                               L.ptr(ones), L.ptr(ones), ctypes.c_float(1.0), L.ptr(st["status"]), st["sms"], land_arr, cnt_arr, 0, w,
                               ctypes.c_uint(state["target"] & 0xFFFFFFFF), L.ptr(shard), 0, ctypes.c_float(1.0), L.ptr(parts), K.NORM_PARTIALS,
                               ctypes.c_uint(5), ctypes.c_double(2.0), L.stream_ptr()), "gemm_rs")

    ms_rs = tm.time(run_rs)
    err = (shard.float() - plain[: M // w].float()).abs().max().item()
    tf = 2.0 * M * N * Kd / 1e9
    out["gemm_rs"] = {"m": M, "n": N, "k": Kd, "ms": round(ms_rs, 4), "tflops": round(tf / ms_rs, 1), "plain_gemm_ms": round(ms_plain, 4),
                      "plain_tflops": round(tf / ms_plain, 1), "max_abs_diff_vs_plain": err,
                      "nvlink_bytes_per_rank": M * N * 2 * (w - 1) // w, "nvlink_ms_at_770GBs": round(M * N * 2 * (w - 1) / w / 770e6, 4)}
    del landing, plain
    # ---- Y = X @ W^T with the rows of W arriving from `w` sources
    M2, N2, K2 = a.rows, a.n2, a.c
    X, W = _rand((M2, K2), f8), _rand((N2, K2), f8)
    Y = torch.empty(M2, N2, dtype=torch.bfloat16, device=DEV)
    flags = torch.full((8,), 3, dtype=torch.int32, device=DEV)
    ms0 = tm.time(lambda: K.gemm(Y, X, W, scale_a=ones, scale_b=ones))
    ms1 = tm.time(lambda: K.gemm(Y, X, W, scale_a=ones, scale_b=ones, ready=(flags.data_ptr(), 3, N2 // w, 2.0)))
    tf2 = 2.0 * M2 * N2 * K2 / 1e9
    out["gemm_ready"] = {"m": M2, "n": N2, "k": K2, "ms": round(ms1, 4), "tflops": round(tf2 / ms1, 1), "plain_gemm_ms": round(ms0, 4),
                         "plain_tflops": round(tf2 / ms0, 1), "nvlink_bytes_per_rank": N2 * K2 * (w - 1) // w,
                         "nvlink_ms_at_770GBs": round(N2 * K2 * (w - 1) / w / 770e6, 4)}
    out[f"{src}_bf16_peak_tflops"] = peak
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["gemm", "gemm_mx", "attention", "elementwise", "adamw", "p2p", "fused_gemm"])
    ap.add_argument("--n2", type=int, default=4608, help="fused_gemm: output columns of the all-gather -> GEMM case (QKV projection)")
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--dtype", default="fp8")
    ap.add_argument("--a-mn", action="store_true")
    ap.add_argument("--b-mn", action="store_true")
    ap.add_argument("--accumulate", action="store_true")
    ap.add_argument("--bias", action="store_true")
    ap.add_argument("--mode", type=int, default=0)
    ap.add_argument("--b", type=int, default=8)
    ap.add_argument("--t", type=int, default=2048)
    ap.add_argument("--hq", type=int, default=28)
    ap.add_argument("--hkv", type=int, default=4)
    ap.add_argument("--hs", type=int, default=128)
    ap.add_argument("--rows", type=int, default=16384)
    ap.add_argument("--c", type=int, default=3584)
    ap.add_argument("--d", type=int, default=18944)
    ap.add_argument("--numel", type=int, default=1 << 28)
    a = ap.parse_args()
    tm = Timer(a.iters, a.warmup, not a.no_flush)
    {"gemm": bench_gemm, "gemm_mx": bench_gemm_mx, "attention": bench_attention, "elementwise": bench_elementwise, "adamw": bench_adamw, "p2p": bench_p2p,
     "fused_gemm": bench_fused_gemm}[a.op](a, tm)


if __name__ == "__main__":
    main()
