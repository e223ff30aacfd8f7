"""Model hyper-parameters: HF ``config.json`` import/export and the built-in table of model names.

Covers the two architectures the reference trains, ``LlamaForCausalLM`` and ``Qwen2ForCausalLM``
(src/training/transformer_config.cpp:13-211).  Qwen2 implies a bias on the fused QKV projection.
"""
from __future__ import annotations

import dataclasses
import json
import os
from dataclasses import dataclass
from typing import Optional

import torch

_DTYPE_NAMES = {
    "fp32": torch.float32, "float32": torch.float32, "f32": torch.float32,
    "bf16": torch.bfloat16, "bfloat16": torch.bfloat16,
    "fp16": torch.float16, "float16": torch.float16, "f16": torch.float16,
    "e4m3": torch.float8_e4m3fn, "fp8": torch.float8_e4m3fn, "float8_e4m3fn": torch.float8_e4m3fn, "f8_e4m3": torch.float8_e4m3fn,
    "e5m2": torch.float8_e5m2, "float8_e5m2": torch.float8_e5m2, "f8_e5m2": torch.float8_e5m2,
    "int32": torch.int32, "i32": torch.int32, "int8": torch.int8, "i8": torch.int8, "byte": torch.uint8, "u8": torch.uint8,
}
_SAFETENSORS_NAMES = {
    torch.float32: "F32", torch.bfloat16: "BF16", torch.float16: "F16", torch.float8_e4m3fn: "F8_E4M3",
    torch.float8_e5m2: "F8_E5M2", torch.int32: "I32", torch.int8: "I8", torch.uint8: "U8", torch.int64: "I64",
}
_SAFETENSORS_REV = {v: k for k, v in _SAFETENSORS_NAMES.items()}


def parse_dtype(name) -> torch.dtype:
    """Accepts the CLI spellings (``bf16``, ``e4m3``, ...), torch names and safetensors names."""
    if isinstance(name, torch.dtype):
        return name
    key = str(name).lower().replace("torch.", "")
    if key in _DTYPE_NAMES:
        return _DTYPE_NAMES[key]
    if str(name).upper() in _SAFETENSORS_REV:
        return _SAFETENSORS_REV[str(name).upper()]
    raise ValueError(f"unknown dtype name {name!r}")


def dtype_to_str(dt: torch.dtype) -> str:
    return {torch.float32: "fp32", torch.bfloat16: "bf16", torch.float16: "fp16", torch.float8_e4m3fn: "e4m3",
            torch.float8_e5m2: "e5m2", torch.int32: "int32", torch.int8: "int8", torch.uint8: "byte"}[dt]


def safetensors_dtype_name(dt: torch.dtype) -> str:
    return _SAFETENSORS_NAMES[dt]


def safetensors_dtype(name: str) -> torch.dtype:
    return _SAFETENSORS_REV[name]


@dataclass
class TransformerConfig:
    architecture: str = "qwen2"            # "qwen2" | "llama"
    bos_token_id: int = 151643
    eos_token_id: int = 151643
    pad_token_id: Optional[int] = None
    hidden_size: int = 896
    intermediate_size: int = 4864
    vocab_size: int = 151936
    num_attention_heads: int = 14
    num_key_value_heads: int = 2
    num_hidden_layers: int = 24
    max_position_embeddings: int = 32768
    rope_theta: float = 1e6
    rms_norm_eps: float = 1e-6
    tie_word_embeddings: bool = True
    use_qkv_bias: bool = True
    dtype: torch.dtype = torch.bfloat16

    # ---- derived sizes
    @property
    def head_size(self) -> int:
        return self.hidden_size // self.num_attention_heads

    @property
    def qkv_channels(self) -> int:
        return (self.num_attention_heads + 2 * self.num_key_value_heads) * self.head_size

    @property
    def model_name(self) -> str:
        return {"qwen2": "Qwen2", "llama": "LLaMA"}[self.architecture]

    @property
    def block_matrix_params(self) -> int:
        C, D = self.hidden_size, self.intermediate_size
        return self.qkv_channels * C + C * C + 2 * D * C + C * D

    def num_parameters(self) -> int:
        C = self.hidden_size
        per_block = self.block_matrix_params + 2 * C + (self.qkv_channels if self.use_qkv_bias else 0)
        emb = self.vocab_size * C
        return self.num_hidden_layers * per_block + emb * (1 if self.tie_word_embeddings else 2) + C

    def validate(self) -> None:
        if self.architecture not in ("qwen2", "llama"):
            raise ValueError(f"unknown architecture {self.architecture}")
        if self.hidden_size % self.num_attention_heads:
            raise ValueError("hidden_size must be divisible by num_attention_heads")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ValueError("num_attention_heads must be divisible by num_key_value_heads")

    # ---- HF interop
    @classmethod
    def from_hf_dict(cls, d: dict, dtype=torch.bfloat16) -> "TransformerConfig":
        archs = d.get("architectures", [])
        if len(archs) != 1:
            raise ValueError("got multiple values for architecture")
        if archs[0] == "LlamaForCausalLM":
            arch = "llama"
        elif archs[0] == "Qwen2ForCausalLM":
            arch = "qwen2"
        else:
            raise ValueError(f"unknown architecture {archs[0]}")
        eos = d["eos_token_id"]
        return cls(
            architecture=arch, bos_token_id=d["bos_token_id"], eos_token_id=eos[0] if isinstance(eos, list) else eos,
            pad_token_id=d.get("pad_token_id"), hidden_size=d["hidden_size"], intermediate_size=d["intermediate_size"],
            vocab_size=d["vocab_size"], num_attention_heads=d["num_attention_heads"],
            num_key_value_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            num_hidden_layers=d["num_hidden_layers"], max_position_embeddings=d["max_position_embeddings"],
            rope_theta=float(d.get("rope_theta", 10000.0)),
            rms_norm_eps=float(d.get("rms_norm_eps", 1e-5 if arch == "llama" else 1e-6)),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)), use_qkv_bias=(arch == "qwen2"),
            dtype=parse_dtype(dtype))

    def to_hf_dict(self) -> dict:
        d = {
            "architectures": ["Qwen2ForCausalLM" if self.architecture == "qwen2" else "LlamaForCausalLM"],
            "model_type": self.architecture,
            "bos_token_id": self.bos_token_id, "eos_token_id": self.eos_token_id,
            "hidden_act": "silu", "hidden_size": self.hidden_size, "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size, "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads, "num_hidden_layers": self.num_hidden_layers,
            "max_position_embeddings": self.max_position_embeddings, "rope_theta": self.rope_theta,
            "rms_norm_eps": self.rms_norm_eps, "tie_word_embeddings": self.tie_word_embeddings,
            "torch_dtype": {torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float16: "float16"}.get(self.dtype, "bfloat16"),
            "attention_dropout": 0.0, "initializer_range": 0.02, "use_cache": True,
        }
        if self.architecture == "qwen2":
            d.update({"use_sliding_window": False, "sliding_window": None, "max_window_layers": self.num_hidden_layers})
        else:
            d.update({"attention_bias": False, "mlp_bias": False})
        if self.pad_token_id is not None:
            d["pad_token_id"] = self.pad_token_id
        return d

    def replace(self, **kw) -> "TransformerConfig":
        return dataclasses.replace(self, **kw)


def load_transformer_config(path: str, dtype=torch.bfloat16) -> TransformerConfig:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    if not os.path.exists(path):
        raise FileNotFoundError(f"could not open config file {path}")
    with open(path) as f:
        return TransformerConfig.from_hf_dict(json.load(f), dtype)


def save_transformer_config(cfg: TransformerConfig, path: str) -> None:
    with open(path, "w") as f:
        json.dump(cfg.to_hf_dict(), f, indent=2)


def _qwen25(h, i, q, kv, depth, eps, tied, dtype, vocab=151936):
    return TransformerConfig("qwen2", 151643, 151643, None, h, i, vocab, q, kv, depth, 32768, 1e6, eps, tied, True, dtype)


def _llama2(h, i, heads, depth, dtype):
    return TransformerConfig("llama", 1, 2, 0, h, i, 32000, heads, heads, depth, 4096, 10000.0, 1e-5, False, False, dtype)


def _llama3(h, i, q, kv, depth, tied, dtype):
    return TransformerConfig("llama", 128000, 128001, 128255, h, i, 128256, q, kv, depth, 4096, 500000.0, 1e-5, tied, False, dtype)


def create_config_from_name(name: str, dtype=torch.bfloat16) -> TransformerConfig:
    """Built-in presets (case-insensitive; an ``org/`` prefix is ignored).

    The larger Qwen2.5 checkpoints ship a 152064-row vocabulary on the hub, which is what the table uses.
    """
    dtype = parse_dtype(dtype)
    key = name.split("/")[-1].lower()
    table = {
        "qwen2.5-0.5b": lambda: _qwen25(896, 4864, 14, 2, 24, 1e-6, True, dtype),
        "qwen2.5-1.5b": lambda: _qwen25(1536, 8960, 12, 2, 28, 1e-6, True, dtype),
        "qwen2.5-3b": lambda: _qwen25(2048, 11008, 16, 2, 36, 1e-6, True, dtype),
        "qwen2.5-7b": lambda: _qwen25(3584, 18944, 28, 4, 28, 1e-6, False, dtype, 152064),
        "qwen2.5-14b": lambda: _qwen25(5120, 13824, 40, 8, 48, 1e-5, False, dtype, 152064),
        "qwen2.5-32b": lambda: _qwen25(5120, 27648, 40, 8, 64, 1e-5, False, dtype, 152064),
        "qwen2.5-72b": lambda: _qwen25(8192, 29568, 64, 8, 80, 1e-5, False, dtype, 152064),
        "llama-2-7b": lambda: _llama2(4096, 11008, 32, 32, dtype),
        "llama-2-13b": lambda: _llama2(5120, 13824, 40, 40, dtype),
        "llama-3-1b": lambda: _llama3(2048, 8192, 32, 8, 16, True, dtype),
        "llama-3.2-1b": lambda: _llama3(2048, 8192, 32, 8, 16, True, dtype),
        "llama-3-3b": lambda: _llama3(3072, 8192, 24, 8, 28, True, dtype),
        "llama-3.2-3b": lambda: _llama3(3072, 8192, 24, 8, 28, True, dtype),
        "llama-3-8b": lambda: _llama3(4096, 14336, 32, 8, 32, False, dtype),
        "llama-3.1-8b": lambda: _llama3(4096, 14336, 32, 8, 32, False, dtype),
        # tiny CPU-test model: 2 layers, hidden 64, 4 q / 2 kv heads, FFN 172, vocab 512, tied, QKV bias
        "tiny-qwen2": lambda: TransformerConfig("qwen2", 0, 0, None, 64, 172, 512, 4, 2, 2, 2048, 1e6, 1e-6, True, True, dtype),
    }
    if key not in table:
        raise ValueError(f"unknown model name {name}")
    return table[key]()
