"""Command-line surface of the trainer: every flag of the reference's ``train`` binary (train.cpp:122-202) and of
its Python front-end (src/binding/python/training.py:14-197), with the same names, defaults and implications,
collected in one dataclass.
"""
from __future__ import annotations

import argparse
import dataclasses
import datetime
from dataclasses import dataclass
from typing import Optional

from ..options import LLamaOptions


@dataclass
class TrainingConfig:
    # model
    model: str = "Qwen2.5-0.5B"
    from_scratch: bool = False
    init_proj_to_zero: bool = False
    model_dtype: str = "bf16"
    matmul_dtype: str = ""
    gradient_dtype: str = ""
    master_dtype: str = ""
    # batch
    batch_size: int = 4
    seq_len: int = 1024
    grad_accumulation: int = 4
    lmhead_chunks: int = 1
    attn_bwd_chunks: int = 1
    # optimiser
    learning_rate: float = 1e-5
    warmup_steps: int = 0
    cooldown_steps: int = 0
    final_lr_fraction: float = 1.0
    lr_schedule: str = "cosine"
    beta_1: float = 0.9
    beta_2: float = 0.95
    opt_m_dtype: str = "fp32"
    opt_v_dtype: str = "fp32"
    grad_clip: float = 1.0
    weight_decay: float = 0.1
    z_loss: float = 0.0
    adam_epsilon: float = 1e-8
    # run length / eval
    steps: int = -1
    epochs: int = 1
    eval_every: int = 100
    eval_num_steps: int = 100
    # data
    train_file: str = "data/train-*.bin"
    train_seed: int = 42
    eval_file: str = "data/eval-*.bin"
    eval_seed: int = 42
    synthetic_data: bool = False
    # output
    name: str = "run"
    out_dir: str = "output/%n"
    checkpoint_dir: str = "ckpt/%n"
    log_file: str = ""
    ckpt_interval: int = 100
    ckpt_keep_n: int = -1
    ckpt_major: int = -1
    save_training_state: bool = True
    continue_from_checkpoint: Optional[str] = None
    new_data: bool = False
    log_gpu_util: int = 25
    verbosity: int = 0
    use_wandb: bool = False
    wandb_project: str = "LLMQ"
    wandb_name: str = ""
    # recompute
    recompute_swiglu: bool = False
    recompute_norm: bool = False
    recompute_ffn: bool = False
    recompute_qkv: bool = False
    recompute_att: bool = False
    recompute_block: bool = False
    offload_residual: bool = False
    # multi-GPU
    gpus: int = 0
    zero_level: int = 0
    shard_weights: bool = False
    shard_gradients: bool = False
    launch: str = "processes"
    # offload
    offload_master: bool = False
    offload_opt_m: bool = False
    offload_opt_v: bool = False
    offload_gradients: bool = False
    persistent_quants: bool = False
    offload_quants: bool = False
    use_zero_copy: bool = False
    write_combined: bool = False
    # algorithms
    memcpy_all_gather: bool = False
    memcpy_send_recv: bool = False
    all_to_all_reduce: bool = False
    use_cuda_graphs: bool = False
    custom_matmul: bool = False
    collectives: str = "auto"
    # debug
    debug_log_allocations: int = 0
    debug_time_breakdown: bool = False
    debug_log_abs_max: int = 0

    def finalize(self) -> "TrainingConfig":
        """Applies %n substitution and the flag relations of the reference (train.cpp:223-250)."""
        for f in ("out_dir", "checkpoint_dir", "log_file"):
            setattr(self, f, getattr(self, f).replace("%n", self.name))
        if not self.log_file:
            stamp = datetime.datetime.now().strftime("%Y%m%d-%H%M%S")
            self.log_file = f"logs/{self.name}-{stamp}.json"
        if self.init_proj_to_zero and not self.from_scratch:
            raise ValueError("--init-proj-to-zero needs --from-scratch")
        if self.zero_level and (self.shard_weights or self.shard_gradients):
            raise ValueError("--zero-level excludes --shard-weights / --shard-gradients")
        if self.zero_level:
            if self.zero_level < 1:
                print("warning: the optimizer state is always sharded; using --zero-level 1")
            self.shard_gradients = self.zero_level >= 2
            self.shard_weights = self.zero_level >= 3
        if self.offload_quants and not self.persistent_quants:
            raise ValueError("--offload-quants needs --persistent-quants")
        if self.persistent_quants and not self.shard_weights:
            raise ValueError("--persistent-quants needs --shard-weights")
        if self.steps > 0 and self.epochs != 1:
            raise ValueError("--steps and --epochs exclude each other")
        return self

    def to_options(self) -> LLamaOptions:
        return LLamaOptions(
            recompute_swiglu=self.recompute_swiglu, recompute_rms_norm=self.recompute_norm, recompute_ffn=self.recompute_ffn,
            recompute_qkv=self.recompute_qkv, recompute_att=self.recompute_att, recompute_block=self.recompute_block,
            offload_residual=self.offload_residual, lmhead_chunks=self.lmhead_chunks, attn_bwd_chunks=self.attn_bwd_chunks,
            use_cuda_graphs=self.use_cuda_graphs, trigger_timing_events=self.debug_time_breakdown, offload_master=self.offload_master,
            offload_quants=self.offload_quants, offload_opt_m=self.offload_opt_m, offload_opt_v=self.offload_opt_v,
            offload_grads=self.offload_gradients, use_zero_copy=self.use_zero_copy, use_write_combined=self.write_combined,
            shard_weights=self.shard_weights, persistent_quants=self.persistent_quants, shard_gradients=self.shard_gradients,
            use_all_to_all_reduce=self.all_to_all_reduce, use_custom_matmul=self.custom_matmul, init_projections_to_zero=self.init_proj_to_zero,
            collectives=self.collectives, memcpy_all_gather=self.memcpy_all_gather, memcpy_send_recv=self.memcpy_send_recv,
            model_type=self.model_dtype, matmul_type=self.matmul_dtype or None, gradient_type=self.gradient_dtype or None,
            master_dtype=self.master_dtype or None, momentum_type=self.opt_m_dtype, variance_type=self.opt_v_dtype)


def add_training_args(p: argparse.ArgumentParser) -> argparse.ArgumentParser:
    d = TrainingConfig()

    def flag(*names, dest, help=""):
        p.add_argument(*names, dest=dest, action="store_true", default=getattr(d, dest), help=help)

    g = p.add_argument_group("model")
    g.add_argument("--model", default=d.model, help="model directory, HF cache name, or built-in preset name")
    flag("--from-scratch", dest="from_scratch", help="random initialisation instead of loading weights")
    flag("--init-proj-to-zero", dest="init_proj_to_zero")
    g.add_argument("--model-dtype", default=d.model_dtype)
    g.add_argument("--matmul-dtype", default=d.matmul_dtype)
    g.add_argument("--gradient-dtype", default=d.gradient_dtype)
    g.add_argument("--master-dtype", default=d.master_dtype)
    g = p.add_argument_group("batch")
    g.add_argument("--batch", "--batch-size", dest="batch_size", type=int, default=d.batch_size, help="per-GPU batch size")
    g.add_argument("--seq-len", "--seq-length", dest="seq_len", type=int, default=d.seq_len)
    g.add_argument("--grad-accumulation", dest="grad_accumulation", type=int, default=d.grad_accumulation)
    g.add_argument("--lmhead-chunks", type=int, default=d.lmhead_chunks)
    g.add_argument("--attn-bwd-chunks", type=int, default=d.attn_bwd_chunks)
    g = p.add_argument_group("optimizer")
    g.add_argument("--lr", "--learning-rate", dest="learning_rate", type=float, default=d.learning_rate)
    g.add_argument("--warmup", dest="warmup_steps", type=int, default=d.warmup_steps)
    g.add_argument("--cooldown", dest="cooldown_steps", type=int, default=d.cooldown_steps)
    g.add_argument("--final-lr-fraction", type=float, default=d.final_lr_fraction)
    g.add_argument("--lr-schedule", choices=["cosine", "linear", "wsd"], default=d.lr_schedule)
    g.add_argument("--beta-1", dest="beta_1", type=float, default=d.beta_1)
    g.add_argument("--beta-2", dest="beta_2", type=float, default=d.beta_2)
    g.add_argument("--opt-m-dtype", default=d.opt_m_dtype)
    g.add_argument("--opt-v-dtype", default=d.opt_v_dtype)
    g.add_argument("--grad-clip", type=float, default=d.grad_clip)
    g.add_argument("--weight-decay", type=float, default=d.weight_decay)
    g.add_argument("--z-loss", type=float, default=d.z_loss)
    g.add_argument("--adam-epsilon", type=float, default=d.adam_epsilon)
    g = p.add_argument_group("run length")
    g.add_argument("--steps", type=int, default=d.steps)
    g.add_argument("--epochs", type=int, default=d.epochs)
    g.add_argument("--eval-every-n-steps", dest="eval_every", type=int, default=d.eval_every)
    g.add_argument("--eval-num-steps", type=int, default=d.eval_num_steps)
    g = p.add_argument_group("data")
    g.add_argument("--train-file", default=d.train_file)
    g.add_argument("--train-seed", type=int, default=d.train_seed)
    g.add_argument("--eval-file", default=d.eval_file)
    g.add_argument("--eval-seed", type=int, default=d.eval_seed)
    flag("--synthetic-data", dest="synthetic_data", help="uniform-random tokens generated in memory (no files needed)")
    g = p.add_argument_group("output")
    g.add_argument("--name", default=d.name)
    g.add_argument("--out-dir", default=d.out_dir)
    g.add_argument("--checkpoint-dir", default=d.checkpoint_dir)
    g.add_argument("--log-file", default=d.log_file)
    g.add_argument("--ckpt-interval", type=int, default=d.ckpt_interval)
    g.add_argument("--ckpt-keep-n", type=int, default=d.ckpt_keep_n)
    g.add_argument("--ckpt-major", type=int, default=d.ckpt_major)
    flag("--save-training-state", dest="save_training_state")
    g.add_argument("--continue", dest="continue_from_checkpoint", nargs="?", const="latest", default=None,
                   help="resume: latest (default), a step number, a step_N directory, or another checkpoint directory")
    flag("--new-data", dest="new_data", help="do not restore the data-loader position")
    g.add_argument("--log-gpu-util", type=int, default=d.log_gpu_util)
    g.add_argument("--verbosity", type=int, default=d.verbosity)
    g.add_argument("-qq", "--silent", dest="verbosity", action="store_const", const=-2, help="no console output")
    g.add_argument("-q", "--quiet", dest="verbosity", action="store_const", const=-1, help="minimal console output")
    g.add_argument("-v", "--verbose", dest="verbosity", action="store_const", const=1, help="detailed console output")
    flag("--use-wandb", dest="use_wandb", help="send every log line to Weights & Biases while training (needs the wandb package)")
    g.add_argument("--wandb-project", default=d.wandb_project)
    g.add_argument("--wandb-name", default=d.wandb_name, help="run name (default: --name)")
    g = p.add_argument_group("recompute")
    for n in ("swiglu", "norm", "ffn", "qkv", "att", "block"):
        flag(f"--recompute-{n}", dest=f"recompute_{n}")
    flag("--offload-residual", dest="offload_residual")
    g = p.add_argument_group("multi-GPU")
    g.add_argument("--gpus", type=int, default=d.gpus, help="0 = all visible GPUs")
    g.add_argument("--zero-level", type=int, default=d.zero_level, choices=[0, 1, 2, 3])
    flag("--shard-weights", dest="shard_weights")
    flag("--shard-gradients", dest="shard_gradients")
    g.add_argument("--launch", choices=["processes", "threads"], default=d.launch,
                   help="how ranks are started when no launcher environment is present")
    g = p.add_argument_group("offload")
    for n in ("master", "opt-m", "opt-v", "gradients", "quants"):
        flag(f"--offload-{n}", dest="offload_" + n.replace("-", "_"))
    flag("--offload-grads", dest="offload_gradients", help="same as --offload-gradients")
    flag("--persistent-quants", dest="persistent_quants")
    flag("--use-zero-copy", dest="use_zero_copy")
    flag("--write-combined", dest="write_combined")
    g = p.add_argument_group("algorithms")
    flag("--memcpy-all-gather", dest="memcpy_all_gather")
    flag("--memcpy-send-recv", dest="memcpy_send_recv")
    flag("--all-to-all-reduce", dest="all_to_all_reduce")
    g.add_argument("--use-cuda-graphs", dest="use_cuda_graphs", action="store_true", default=d.use_cuda_graphs)
    g.add_argument("--no-use-cuda-graphs", dest="use_cuda_graphs", action="store_false")
    flag("--custom-matmul", dest="custom_matmul")
    g.add_argument("--collectives", choices=["auto", "fused", "nccl"], default=d.collectives)
    g = p.add_argument_group("debug")
    g.add_argument("--debug-log-allocations", type=int, default=d.debug_log_allocations)
    flag("--debug-time-breakdown", dest="debug_time_breakdown")
    g.add_argument("--debug-log-abs-max", type=int, default=d.debug_log_abs_max)
    return p


def parse_training_config(argv=None) -> TrainingConfig:
    p = add_training_args(argparse.ArgumentParser(description="Train a Llama / Qwen2 decoder"))
    ns = p.parse_args(argv)
    fields = {f.name for f in dataclasses.fields(TrainingConfig)}
    return TrainingConfig(**{k: v for k, v in vars(ns).items() if k in fields}).finalize()
