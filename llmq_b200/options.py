"""Run-time options of the trainer (what the ``train`` flags and the Python API set).

Field names follow the Python binding of the reference (src/binding/binding.cpp:149-238,
src/models/llama_model.h:22-58) so that scripts written against it keep working.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from .config import parse_dtype


@dataclass
class LLamaOptions:
    # activation recomputation
    recompute_swiglu: bool = False
    recompute_rms_norm: bool = False
    recompute_ffn: bool = False
    recompute_qkv: bool = False
    recompute_att: bool = False
    recompute_block: bool = False
    offload_residual: bool = False
    lmhead_chunks: int = 1
    attn_bwd_chunks: int = 1
    use_cuda_graphs: bool = False
    # weight-gradient GEMMs of the blocks on a second stream, beside the element-wise kernels of the dX chain.  It paid while
    # those GEMMs read MN-major operands and left the tensor pipe half idle (-10 ms per 7B step); with K-major operands they
    # fill the SMs themselves and sharing costs more than it hides (477.7 ms off against 481-485 ms on, same box), so: off.
    overlap_dw: bool = False
    overlap_lmhead: bool = True               # LM-head gradient GEMMs of a chunk on the second stream, beside the next chunk's logits + classifier
    # bit 0 / 1: SwiGLU forward / backward inside GEMM epilogues (GPU, bf16 activations).  Bit-identical to the separate
    # kernels; off by default: with four epilogue warps per CTA the extra math takes as long as the memory pass it saves
    # (Qwen2.5-7B step: 495.6 ms without, 494.3 forward only, 498.9 backward only, 497.8 both).
    fuse_swiglu: int = 0
    # block-scaled (MX) e4m3 matmuls: every GEMM operand of the transformer blocks is quantised with one power-of-two scale
    # per 32 elements of the contraction axis (tcgen05 kind::mxf8f6f4.block_scale); activations and weights stay bf16.
    # Also selected by matmul_type = "mxe4m3" / "mxfp8".
    block_scaled: bool = False
    swiglu_backward_two_pass: bool = True     # fp8 K-major backward: SwiGLU gradient as abs-max pass + quantise/transpose pass, its bf16 form never stored
    # ZeRO-3: start the next block's weight gather behind the current block's first GEMM(s), beside attention, instead of at the
    # top of the block (each block body then runs as two graphs).  Off: no gain measured on 2 GPUs (481.3 / 485.2 ms off, 483.9 /
    # 482.8 ms on; the pushes need most SMs to fill NVLink - limited to 16 SMs the step took 492-507 ms).
    gather_behind_first_gemm: bool = False
    kmajor_backward: bool = True              # fp8 backward GEMMs read transposed fp8 copies (all operands K-major) instead of MN-major tiles
    lmhead_transposed_operands: bool = True   # LM-head backward reads W^T / lnf^T copies (K-major GEMM operands)
    # ... and a transposed copy of each d(logits) chunk for the dW GEMM: no measurable gain (469.3 / 472.4 ms with, 472.1 / 470.7 ms
    # without, same box) for 1.25 GB more, so off
    lmhead_transpose_dlogits: bool = False
    trigger_timing_events: bool = False
    # placement of state
    offload_master: bool = False
    offload_quants: bool = False
    offload_opt_m: bool = False
    offload_opt_v: bool = False
    offload_grads: bool = False
    use_zero_copy: bool = False
    use_write_combined: bool = False
    # sharding
    shard_weights: bool = False
    persistent_quants: bool = False
    shard_gradients: bool = False
    use_all_to_all_reduce: bool = False
    use_custom_matmul: bool = False          # accepted for compatibility: every GEMM already is the in-tree tcgen05 kernel
    init_projections_to_zero: bool = False
    # collectives: "fused" = in-kernel NVLink peer loads/stores, "nccl" = library collectives on a side stream
    collectives: str = "auto"
    memcpy_all_gather: bool = False
    memcpy_send_recv: bool = False
    # dtypes (None -> derived)
    model_type: Optional[torch.dtype] = None
    matmul_type: Optional[torch.dtype] = None
    gradient_type: Optional[torch.dtype] = None
    master_dtype: Optional[torch.dtype] = None
    momentum_type: torch.dtype = torch.float32
    variance_type: torch.dtype = torch.float32

    def __post_init__(self):
        if isinstance(self.matmul_type, str) and self.matmul_type.lower() in ("mxe4m3", "mxfp8", "mx"):
            self.block_scaled, self.matmul_type = True, None
        for name in ("model_type", "matmul_type", "gradient_type", "master_dtype", "momentum_type", "variance_type"):
            v = getattr(self, name)
            if v is not None and v != "" and not isinstance(v, torch.dtype):
                setattr(self, name, parse_dtype(v))
            elif v == "":
                setattr(self, name, None)
        self.apply_implications()

    # the reference spells this option both ways in its Python binding
    @property
    def recompute_rmsnorm(self) -> bool:
        return self.recompute_rms_norm

    @recompute_rmsnorm.setter
    def recompute_rmsnorm(self, v: bool) -> None:
        self.recompute_rms_norm = v

    def apply_implications(self) -> None:
        """recompute-block => att, ffn, norm;  att => qkv;  ffn => swiglu (train.cpp:239-250 of the reference)."""
        if self.recompute_block:
            self.recompute_att = self.recompute_ffn = self.recompute_rms_norm = True
        if self.recompute_att:
            self.recompute_qkv = True
        if self.recompute_ffn:
            self.recompute_swiglu = True
        if self.offload_quants and not self.persistent_quants:
            raise ValueError("offload_quants requires persistent_quants")
        if self.persistent_quants and not self.shard_weights:
            raise ValueError("persistent_quants requires shard_weights")

    def matmul_dtype(self) -> torch.dtype:
        return self.matmul_type or self.model_type or torch.bfloat16

    def grad_dtype(self) -> torch.dtype:
        return self.gradient_type or self.matmul_dtype()

    def master(self) -> torch.dtype:
        return self.master_dtype or self.model_type or torch.bfloat16

    def set_zero_level(self, level: int) -> None:
        """1 = sharded optimizer state (always on), 2 = + sharded gradients, 3 = + sharded weights."""
        if level < 1:
            level = 1
        self.shard_gradients = level >= 2
        self.shard_weights = level >= 3
