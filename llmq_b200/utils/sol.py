"""Speed-of-light (SOL / MFU) estimate: time per token if every matmul ran at the GPU's peak.

Same definition as the reference (src/utilities/sol.cpp:292-321): 6 * block-matrix parameters in the matmul
dtype + 6 * V * C (LM head) in the model dtype + 6 * L * (Hq*HS) * T (attention) in the model dtype, each divided
by the peak throughput of its dtype, divided by the world size.  Two denominators are offered: the spec-sheet
table (dense, no sparsity) and a measured bf16 peak (``measure_real_peak`` runs the in-tree tcgen05 GEMM).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional

import torch

# dense TFLOP/s by dtype family
GPU_SPECS: Dict[str, Dict[str, float]] = {
    "NVIDIA B200": {"bf16": 2200.0, "fp8": 4500.0, "fp4": 9000.0, "fp32": 1100.0},
    "NVIDIA B100": {"bf16": 1800.0, "fp8": 3500.0, "fp4": 7000.0, "fp32": 900.0},
    "NVIDIA H100 80GB HBM3": {"bf16": 989.0, "fp8": 1979.0, "fp32": 494.0},
    "NVIDIA H100 PCIe": {"bf16": 756.0, "fp8": 1513.0, "fp32": 378.0},
    "NVIDIA H200": {"bf16": 989.0, "fp8": 1979.0, "fp32": 494.0},
    "NVIDIA A100-SXM4-80GB": {"bf16": 312.0, "fp8": 312.0, "fp32": 156.0},
    "NVIDIA L40S": {"bf16": 362.0, "fp8": 733.0, "fp32": 183.0},
    "NVIDIA RTX PRO 6000 Blackwell Server Edition": {"bf16": 503.0, "fp8": 1007.0, "fp32": 126.0},
    "NVIDIA GeForce RTX 5090": {"bf16": 209.5, "fp8": 419.0, "fp32": 104.8},
    "NVIDIA GeForce RTX 4090": {"bf16": 165.2, "fp8": 330.3, "fp32": 82.6},
}


def _family(dt: torch.dtype) -> str:
    if dt in (torch.float8_e4m3fn, torch.float8_e5m2):
        return "fp8"
    if dt == torch.float32:
        return "fp32"
    return "bf16"


def get_gpu_spec(name: str) -> Optional[Dict[str, float]]:
    if name in GPU_SPECS:
        return GPU_SPECS[name]
    for k, v in GPU_SPECS.items():
        if k in name or name in k:
            return v
    return None


@dataclass
class TransformerOps:
    block_flop: float        # per token, in the matmul dtype
    head_flop: float         # per token, in the model dtype
    attention_flop: float    # per token, in the model dtype


def get_transformer_ops(cfg, seq_len: int) -> TransformerOps:
    C = cfg.hidden_size
    return TransformerOps(6.0 * cfg.num_hidden_layers * cfg.block_matrix_params, 6.0 * cfg.vocab_size * C,
                          6.0 * cfg.num_hidden_layers * (cfg.num_attention_heads * cfg.head_size) * seq_len)


def estimate_speed_of_light(cfg, seq_len: int, model_dtype: torch.dtype, matmul_dtype: torch.dtype, world: int = 1,
                            gpu_name: str = "NVIDIA B200", peaks: Optional[Dict[str, float]] = None) -> float:
    """Nanoseconds per token at peak throughput (whole job, i.e. already divided by the world size)."""
    spec = peaks or get_gpu_spec(gpu_name)
    if spec is None:
        return 0.0
    ops = get_transformer_ops(cfg, seq_len)
    mm, md = spec[_family(matmul_dtype)], spec[_family(model_dtype)]
    ns = ops.block_flop / (mm * 1e12) * 1e9 + (ops.head_flop + ops.attention_flop) / (md * 1e12) * 1e9
    return ns / max(1, world)


def measure_real_peak(seconds: float = 0.5, n: int = 8192) -> float:
    """Sustained bf16 TFLOP/s of an n^3 GEMM on the current device, run back to back for ``seconds``."""
    from ..ops import kernels as K
    dev = torch.device("cuda", torch.cuda.current_device())
    a = torch.randn(n, n, device=dev).bfloat16()
    b = torch.randn(n, n, device=dev).bfloat16()
    c = torch.empty(n, n, device=dev, dtype=torch.bfloat16)
    for _ in range(3):
        K.gemm(c, a, b)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    iters, total_ms = 0, 0.0
    while total_ms < seconds * 1e3:
        e0.record()
        for _ in range(10):
            K.gemm(c, a, b)
        e1.record()
        torch.cuda.synchronize()
        total_ms += e0.elapsed_time(e1)
        iters += 10
    return 2.0 * n ** 3 * iters / (total_ms / 1e3) / 1e12
