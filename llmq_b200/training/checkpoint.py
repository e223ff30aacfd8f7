"""Sharded training checkpoints.

Layout (directory structure of the reference, src/training/checkpoint.cpp:24-189, src/models/llama_optimizer.cpp:55-79):

    <dir>/step_00000100/weights.shard_000_of_008.safetensors     master-weight shards, fused names
                        adam.m.shard_000_of_008.safetensors      first moments (+ adam.m.scales.* for e4m3)
                        adam.v.shard_000_of_008.safetensors
                        checkpoint.json                          {version, data-loader, run, distributed}

The directory layout, the shard file names and the top-level keys of ``checkpoint.json`` are the reference's; the values
under ``run`` are not interchangeable with it: the random state is one decimal number here (a byte vector there), the
outlier windows are flat lists (``past_losses.values / index / size`` there), and the step counter of the gradient manager
and the stochastic-rounding state are stored in addition.  Checkpoints are therefore portable between runs of this
framework only; the HF export (``model.safetensors``) is the interchange format.

Every rank writes its own shard files (tmp + rename), then rank 0 writes ``checkpoint.json`` last, so a directory
with that file is complete.  Restoring needs the same world size; corrupted, truncated or mismatching shards
raise instead of loading silently.
"""
from __future__ import annotations

import json
import os
import re
import shutil
from typing import Dict, List, Optional

import torch

from ..utils.hf_io import checkpoint_name
from ..utils.safetensors import SafeTensorsReader, SafeTensorsWriter

CHECKPOINT_VERSION = 20260120


def get_checkpoint_path(directory: str, step: int) -> str:
    return os.path.join(directory, f"step_{step:08d}")


def get_all_checkpoints(directory: str) -> List[int]:
    if not os.path.isdir(directory):
        return []
    steps = []
    for d in os.listdir(directory):
        m = re.fullmatch(r"step_(\d{8})", d)
        if m and os.path.exists(os.path.join(directory, d, "checkpoint.json")):
            steps.append(int(m.group(1)))
    return sorted(steps)


def find_latest_checkpoint(directory: str) -> int:
    steps = get_all_checkpoints(directory)
    return steps[-1] if steps else -1


def clean_old_checkpoints(directory: str, keep_n: int, major_every: int = -1) -> List[int]:
    """Removes old checkpoints like the reference (src/training/checkpoint.cpp:170-189): nothing happens while at most
    ``keep_n`` checkpoints exist; otherwise the steps divisible by ``major_every`` are set aside (never removed) and of the
    remaining ones only the newest ``keep_n`` survive.  Returns the removed steps."""
    steps = get_all_checkpoints(directory)
    if keep_n <= 0 or len(steps) <= keep_n:
        return []
    if major_every > 0:
        steps = [s for s in steps if s % major_every != 0]
    removed = []
    for s in sorted(steps)[:max(0, len(steps) - keep_n)]:
        shutil.rmtree(get_checkpoint_path(directory, s), ignore_errors=True)
        removed.append(s)
    return removed


def _shard_file(path: str, kind: str, rank: int, world: int) -> str:
    return os.path.join(path, f"{kind}.shard_{rank:03d}_of_{world:03d}.safetensors")


def _write_shards(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    w = SafeTensorsWriter(path)
    for n, t in tensors.items():
        w.register(n, t.dtype, t.shape)
    w.prepare(True)
    for n, t in tensors.items():
        w.write(n, t)
    w.finalize(True)


def save_checkpoint(directory: str, step: int, model, extra: Optional[dict] = None) -> str:
    """``extra`` may carry {"data-loader": {...}, "run": {...}}; returns the checkpoint path."""
    comm = model.comm
    path = get_checkpoint_path(directory, step)
    if comm.rank == 0:
        os.makedirs(path, exist_ok=True)
        stale = os.path.join(path, "checkpoint.json")
        if os.path.exists(stale):
            os.remove(stale)                     # the marker goes first, so a half-overwritten directory is not "complete"
    comm.barrier()
    r, w = comm.rank, comm.world
    weights = {checkpoint_name(n): t for n, t, _, _ in model.weights.master_items()}
    _write_shards(_shard_file(path, "weights", r, w), weights)
    opt = model.opt_state
    _write_shards(_shard_file(path, "adam.m", r, w), {checkpoint_name(n): t for n, t in opt.m.items()})
    _write_shards(_shard_file(path, "adam.v", r, w), {checkpoint_name(n): t for n, t in opt.v.items()})
    if opt.m_scales:
        _write_shards(_shard_file(path, "adam.m.scales", r, w), {checkpoint_name(n): t for n, t in opt.m_scales.items()})
    comm.barrier()
    if comm.rank == 0:
        extra = extra or {}
        meta = {
            "version": CHECKPOINT_VERSION,
            "data-loader": extra.get("data-loader", {}),
            "run": {"step": step, "rng": str(model.rng_state), "grad_step": model.grads.step, **extra.get("run", {})},
            "distributed": {"world": w},
        }
        tmp = os.path.join(path, "checkpoint.json.tmp")
        with open(tmp, "w") as f:
            json.dump(meta, f, indent=2)
        os.replace(tmp, os.path.join(path, "checkpoint.json"))
    comm.barrier()
    return path


def _read_shards(path: str, tensors: Dict[str, torch.Tensor]) -> None:
    if not os.path.exists(path):
        raise FileNotFoundError(f"checkpoint shard {path} is missing")
    r = SafeTensorsReader(path)
    for n, t in tensors.items():
        if n not in r:
            raise KeyError(f"{path}: tensor {n} missing")
        e = r.entries[n]
        if tuple(e.shape) != tuple(t.shape) or e.dtype != t.dtype:
            raise ValueError(f"{path}: tensor {n} is {e.dtype}{tuple(e.shape)}, expected {t.dtype}{tuple(t.shape)}")
        if t.device.type == "cpu":
            r.read_into(n, t)
        else:
            r.read_into(n, t)


def load_checkpoint(directory: str, step: int, model) -> dict:
    """Restores master weights, Adam moments and the stochastic-rounding state; returns the parsed ``checkpoint.json``."""
    comm = model.comm
    path = directory if os.path.exists(os.path.join(directory, "checkpoint.json")) else get_checkpoint_path(directory, step)
    meta_file = os.path.join(path, "checkpoint.json")
    if not os.path.exists(meta_file):
        raise FileNotFoundError(f"{path} is not a complete checkpoint (checkpoint.json missing)")
    with open(meta_file) as f:
        meta = json.load(f)
    if meta.get("version") != CHECKPOINT_VERSION:
        raise ValueError(f"checkpoint version {meta.get('version')} is not supported (expected {CHECKPOINT_VERSION})")
    world = meta.get("distributed", {}).get("world")
    if world != comm.world:
        raise ValueError(f"checkpoint was written with world size {world}, this run has {comm.world}")
    r, w = comm.rank, comm.world
    _read_shards(_shard_file(path, "weights", r, w), {checkpoint_name(n): t for n, t, _, _ in model.weights.master_items()})
    opt = model.opt_state
    _read_shards(_shard_file(path, "adam.m", r, w), {checkpoint_name(n): t for n, t in opt.m.items()})
    _read_shards(_shard_file(path, "adam.v", r, w), {checkpoint_name(n): t for n, t in opt.v.items()})
    if opt.m_scales:
        _read_shards(_shard_file(path, "adam.m.scales", r, w), {checkpoint_name(n): t for n, t in opt.m_scales.items()})
    run = meta.get("run", {})
    model.rng_state = int(run.get("rng", model.rng_state))
    model.grads.step = int(run.get("grad_step", 0))
    model.on_weights_changed()
    comm.barrier()
    return meta
