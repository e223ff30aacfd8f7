"""Hugging Face weight import / export for the fused parameter layout.

Import fuses ``q_proj/k_proj/v_proj`` row-wise into ``qkv`` and ``up_proj/gate_proj`` into ``up`` (up first);
export splits them back, so the written ``model.safetensors`` + ``config.json`` load in ``transformers``
(reference: src/models/llama_weights.cpp:915-1043).  Every rank touches only the rows of its own shard:
on import it reads the intersecting row ranges straight into its master shard, on export all ranks write
their byte ranges into one shared memory-mapped file (works with one process per GPU, not only with threads).
"""
from __future__ import annotations

import os
import shutil
from typing import Dict, List, Tuple

import torch

from ..config import save_transformer_config
from .safetensors import SafeTensorsReader, SafeTensorsWriter

# internal name -> checkpoint (fused) name
CKPT_BLOCK_NAMES = {
    "ln1_w": "model.layers.{l}.input_layernorm.weight",
    "qkv_w": "model.layers.{l}.self_attn.qkv.weight",
    "qkv_b": "model.layers.{l}.self_attn.qkv.bias",
    "o_w": "model.layers.{l}.self_attn.o_proj.weight",
    "ln2_w": "model.layers.{l}.post_attention_layernorm.weight",
    "up_w": "model.layers.{l}.mlp.up.weight",
    "down_w": "model.layers.{l}.mlp.down_proj.weight",
}
CKPT_NB_NAMES = {"embed": "model.embed_tokens.weight", "lnf_w": "model.norm.weight", "lm_head": "lm_head.weight"}


def checkpoint_name(internal: str) -> str:
    """``layers.3.qkv_w`` -> ``model.layers.3.self_attn.qkv.weight``."""
    if internal.startswith("layers."):
        _, l, n = internal.split(".", 2)
        return CKPT_BLOCK_NAMES[n].format(l=l)
    return CKPT_NB_NAMES[internal]


def hf_parts(cfg, internal: str) -> List[Tuple[str, int]]:
    """HF tensors (name, rows) that are concatenated along dim 0 to form the internal tensor."""
    HS, Hq, Hkv, D = cfg.head_size, cfg.num_attention_heads, cfg.num_key_value_heads, cfg.intermediate_size
    if internal.startswith("layers."):
        _, l, n = internal.split(".", 2)
        pre = f"model.layers.{l}."
        if n in ("qkv_w", "qkv_b"):
            suf = "weight" if n == "qkv_w" else "bias"
            return [(pre + f"self_attn.q_proj.{suf}", Hq * HS), (pre + f"self_attn.k_proj.{suf}", Hkv * HS), (pre + f"self_attn.v_proj.{suf}", Hkv * HS)]
        if n == "up_w":
            return [(pre + "mlp.up_proj.weight", D), (pre + "mlp.gate_proj.weight", D)]
        single = {"ln1_w": "input_layernorm.weight", "o_w": "self_attn.o_proj.weight", "ln2_w": "post_attention_layernorm.weight",
                  "down_w": "mlp.down_proj.weight"}[n]
        rows = cfg.hidden_size
        return [(pre + single, rows)]
    if internal == "embed":
        return [("model.embed_tokens.weight", cfg.vocab_size)]
    if internal == "lnf_w":
        return [("model.norm.weight", cfg.hidden_size)]
    if internal == "lm_head":
        return [("lm_head.weight", cfg.vocab_size)]
    raise KeyError(internal)


def _row_elems(t: torch.Tensor) -> int:
    return t.numel() // max(t.shape[0], 1)


def import_hf_weights(model, path: str) -> None:
    """Fills the master shards of ``model`` from an HF checkpoint directory / file."""
    reader = SafeTensorsReader(path)
    rank = model.comm.rank
    for name, master, spec, l in model.weights.master_items():
        rows = master.shape[0]
        a, b = rank * rows, (rank + 1) * rows
        per_row = _row_elems(master)
        dev = master if master.device.type == model.device.type else torch.empty(master.shape, dtype=master.dtype, device=model.device)
        flat = dev.view(-1)
        start = 0
        for hf_name, part_rows in hf_parts(model.cfg, name):
            lo, hi = max(a, start), min(b, start + part_rows)
            if lo < hi:
                src_name = hf_name
                if src_name not in reader and hf_name == "lm_head.weight":
                    src_name = "model.embed_tokens.weight"        # checkpoints of tied models omit the head
                dst = flat[(lo - a) * per_row:(hi - a) * per_row]
                reader.read_into(src_name, dst, elem_offset=(lo - start) * per_row)
            start += part_rows
        if dev is not master:
            master.copy_(dev)
    model.on_weights_changed()


def export_hf_model(model, out_dir: str, source_dir: str = None) -> None:
    """Writes ``config.json`` + a single ``model.safetensors`` with HF names (q/k/v and up/gate split)."""
    comm, cfg = model.comm, model.cfg
    os.makedirs(out_dir, exist_ok=True)
    path = os.path.join(out_dir, "model.safetensors")
    w = SafeTensorsWriter(path)
    layout: Dict[str, List[Tuple[str, int]]] = {}
    for name, master, spec, l in model.weights.master_items():
        parts = hf_parts(cfg, name)
        layout[name] = parts
        full_tail = tuple(master.shape[1:])
        for hf_name, rows in parts:
            w.register(hf_name, master.dtype, (rows,) + full_tail)
    if comm.rank == 0:
        w.prepare(create=True)
        save_transformer_config(cfg.replace(dtype=model.weights.master_dtype), os.path.join(out_dir, "config.json"))
    comm.barrier()
    if comm.rank != 0:
        w.prepare(create=False)
    for name, master, spec, l in model.weights.master_items():
        rows = master.shape[0]
        a, b = comm.rank * rows, (comm.rank + 1) * rows
        per_row_bytes = _row_elems(master) * master.element_size()
        src = master if master.device.type == model.device.type else master       # host shards are written directly
        flat = src.reshape(rows, -1)
        start = 0
        for hf_name, part_rows in layout[name]:
            lo, hi = max(a, start), min(b, start + part_rows)
            if lo < hi:
                w.write_raw(hf_name, flat[lo - a:hi - a], byte_offset=(lo - start) * per_row_bytes)
            start += part_rows
    comm.barrier()
    w.finalize(rename=comm.rank == 0)
    if comm.rank == 0 and source_dir and os.path.isdir(source_dir):
        for fn in os.listdir(source_dir):                          # tokenizer files travel with the model
            if fn.startswith("tokenizer") or fn in ("vocab.json", "merges.txt", "special_tokens_map.json", "generation_config.json"):
                shutil.copy(os.path.join(source_dir, fn), os.path.join(out_dir, fn))
    comm.barrier()
