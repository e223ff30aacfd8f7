"""``export-checkpoint``: turns a sharded training checkpoint into an HF-loadable ``model.safetensors`` + ``config.json``.

Flags of the reference tool (export-checkpoint.cpp:34-41): ``--model --checkpoint-dir --out-dir`` (+ dtype options,
accepted for compatibility).  No GPU and no process group are needed: the shards of all ranks recorded in the
checkpoint are read tensor by tensor, joined along dimension 0, split into the HF tensors and streamed into the
output file.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

from ..config import create_config_from_name, load_transformer_config, save_transformer_config
from ..options import LLamaOptions
from ..parallel.zero import block_param_specs, nonblock_param_specs
from ..training import checkpoint as ck
from ..utils.hf_io import checkpoint_name, hf_parts
from ..utils.safetensors import SafeTensorsReader, SafeTensorsWriter, resolve_model_dir


def export_checkpoint(model: str, checkpoint_dir: str, out_dir: str, step: int = -1, model_dtype: str = "bf16") -> str:
    try:
        cfg = load_transformer_config(resolve_model_dir(model), model_dtype)
    except FileNotFoundError:
        cfg = create_config_from_name(model, model_dtype)
    if os.path.exists(os.path.join(checkpoint_dir, "checkpoint.json")):
        path = checkpoint_dir
    else:
        if step < 0:
            step = ck.find_latest_checkpoint(checkpoint_dir)
        if step < 0:
            raise FileNotFoundError(f"no checkpoint found in {checkpoint_dir}")
        path = ck.get_checkpoint_path(checkpoint_dir, step)
    with open(os.path.join(path, "checkpoint.json")) as f:
        world = json.load(f)["distributed"]["world"]
    readers = [SafeTensorsReader(os.path.join(path, f"weights.shard_{r:03d}_of_{world:03d}.safetensors")) for r in range(world)]
    names = [f"layers.{l}.{s.name}" for l in range(cfg.num_hidden_layers) for s in block_param_specs(cfg, LLamaOptions())]
    names += [s.name for s in nonblock_param_specs(cfg)]
    os.makedirs(out_dir, exist_ok=True)
    w = SafeTensorsWriter(os.path.join(out_dir, "model.safetensors"))
    dtype = None
    for n in names:
        e = readers[0].entries[checkpoint_name(n)]
        dtype = e.dtype
        tail = tuple(e.shape[1:])
        for hf_name, rows in hf_parts(cfg, n):
            w.register(hf_name, e.dtype, (rows,) + tail)
    w.prepare(True)
    for n in names:
        full = torch.cat([r.read(checkpoint_name(n)) for r in readers], 0)
        start = 0
        for hf_name, rows in hf_parts(cfg, n):
            w.write(hf_name, full[start:start + rows].contiguous())
            start += rows
    w.finalize(True)
    save_transformer_config(cfg.replace(dtype=dtype or cfg.dtype), os.path.join(out_dir, "config.json"))
    return out_dir


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="Export the latest checkpoint as an HF model")
    p.add_argument("--model", required=True)
    p.add_argument("--checkpoint-dir", required=True)
    p.add_argument("--out-dir", required=True)
    p.add_argument("--step", type=int, default=-1)
    p.add_argument("--model-dtype", default="bf16")
    p.add_argument("--opt-m-dtype", default="fp32")
    p.add_argument("--opt-v-dtype", default="fp32")
    a = p.parse_args(argv)
    out = export_checkpoint(a.model, a.checkpoint_dir, a.out_dir, a.step, a.model_dtype)
    print(f"exported to {out}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
