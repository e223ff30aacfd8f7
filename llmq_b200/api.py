"""Python API with the surface of the reference's ``pyllmq`` module (src/binding/binding.cpp:46-456):
``Config``, ``LLamaOptions``, ``LLMQTrainer`` plus the helpers re-exported from the sub-modules.

``LLMQTrainer`` drives one model replica per GPU:

* ``ngpu == 1`` (or a launcher environment with one rank per process, e.g. ``torchrun``): the trainer of this
  process owns one GPU and takes part in the collectives of its process group.  ``step`` accepts either the
  local ``(B, T)`` token block or the global ``(world * B, T)`` array, from which the rank takes its rows.
* ``ngpu > 1`` inside a single Python process: one worker per GPU is started (``parallel/launcher.py``) and
  ``step`` splits the ``(ngpu * B, T)`` arrays by rank, like MultiGPUPyTrainer (src/binding/py_train.cpp:97-118).
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import numpy as np
import torch

from .config import TransformerConfig, create_config_from_name, load_transformer_config, parse_dtype
from .options import LLamaOptions


class Config(TransformerConfig):
    """``TransformerConfig`` with the constructor spellings of the reference binding."""

    def __init__(self, architecture="qwen2", hidden_size=896, intermediate_size=4864, num_attention_heads=14,
                 num_key_value_heads=2, num_hidden_layers=24, rms_norm_eps=1e-6, tie_word_embeddings=True,
                 bos_token_id=151643, eos_token_id=151643, pad_token_id=None, vocab_size=151936,
                 max_position_embeddings=32768, rope_theta=1e6, use_qkv_bias=None, dtype="bf16"):
        arch = architecture.lower()
        super().__init__(architecture=arch, bos_token_id=bos_token_id, eos_token_id=eos_token_id, pad_token_id=pad_token_id,
                         hidden_size=hidden_size, intermediate_size=intermediate_size, vocab_size=vocab_size,
                         num_attention_heads=num_attention_heads, num_key_value_heads=num_key_value_heads,
                         num_hidden_layers=num_hidden_layers, max_position_embeddings=max_position_embeddings,
                         rope_theta=rope_theta, rms_norm_eps=rms_norm_eps, tie_word_embeddings=tie_word_embeddings,
                         use_qkv_bias=(arch == "qwen2") if use_qkv_bias is None else use_qkv_bias, dtype=parse_dtype(dtype))

    @staticmethod
    def from_name(name: str, dtype="bf16") -> TransformerConfig:
        return create_config_from_name(name, dtype)

    @staticmethod
    def from_pretrained(name: str, dtype="bf16") -> TransformerConfig:
        from .utils.safetensors import resolve_model_dir
        try:
            return load_transformer_config(resolve_model_dir(name), dtype)
        except FileNotFoundError:
            return create_config_from_name(name, dtype)


def get_num_gpus() -> int:
    return torch.cuda.device_count()


def _as_tensor(a) -> torch.Tensor:
    if isinstance(a, torch.Tensor):
        return a
    return torch.from_numpy(np.ascontiguousarray(a))


class LLMQTrainer:
    def __init__(self, ngpu: Optional[int] = None, config: Optional[TransformerConfig] = None, options: Optional[LLamaOptions] = None,
                 batch_size: int = 4, seq_len: int = 1024, grad_accum: int = 1, memcpy_all_gather: bool = False,
                 memcpy_send_recv: bool = False, device: Optional[str] = None):
        from .models.llama import LlamaModel
        from .parallel.comm import LocalComm, make_communicator

        self.config = config
        self.options = options or LLamaOptions()
        self.options.memcpy_all_gather = memcpy_all_gather
        self.options.memcpy_send_recv = memcpy_send_recv
        self.batch_size, self.seq_length, self.grad_accum = batch_size, seq_len, grad_accum
        from .parallel.threads import current_thread_comm
        tcomm = current_thread_comm()                 # set when this rank runs as a thread of a multi-rank process
        env_world = tcomm.world if tcomm is not None else int(os.environ.get("WORLD_SIZE", os.environ.get("OMPI_COMM_WORLD_SIZE", "1")))
        self._pool = None
        if ngpu is None or ngpu <= 0:
            ngpu = env_world if env_world > 1 else 1
        self.world_size = ngpu
        if ngpu > 1 and env_world == 1:
            from .parallel.launcher import WorkerPool
            self._pool = WorkerPool(ngpu, config, self.options, batch_size, seq_len, grad_accum,
                                    use_cuda=None if device is None else device != "cpu")
            self.model = None
            self.rank = 0
            self._micro = 0
            return
        if tcomm is not None and device is None:
            device = str(tcomm.device)
        if device is None:
            if torch.cuda.is_available():
                local = int(os.environ.get("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", "0")))
                torch.cuda.set_device(local)
                device = f"cuda:{local}"
            else:
                device = "cpu"
        self.device = torch.device(device)
        if tcomm is not None:
            self.comm = tcomm
        else:
            self.comm = make_communicator(self.device) if env_world > 1 else LocalComm()
        if ngpu != self.comm.world:
            raise ValueError(f"ngpu={ngpu} does not match the launcher's world size {self.comm.world}")
        self.rank = self.comm.rank
        self.model = LlamaModel(config, self.options, self.comm, self.device, batch_size, seq_len)
        self._micro = 0
        pin = self.device.type == "cuda"
        self._in_pinned = torch.zeros(batch_size, seq_len, dtype=torch.int32, pin_memory=pin)
        self._tg_pinned = torch.zeros(batch_size, seq_len, dtype=torch.int32, pin_memory=pin)
        self._copied = torch.cuda.Event() if pin else None
        self._copy_pending = False

    # ------------------------------------------------------------------ construction helpers
    @classmethod
    def from_pretrained(cls, name: str, ngpu: int = 1, dtype="bf16", options: Optional[LLamaOptions] = None, batch_size: int = 4,
                        seq_len: int = 1024, grad_accum: int = 1, memcpy_all_gather: bool = False, memcpy_send_recv: bool = False):
        from .utils.safetensors import resolve_model_dir
        path = resolve_model_dir(name)
        cfg = load_transformer_config(path, dtype)
        tr = cls(ngpu, cfg, options, batch_size, seq_len, grad_accum, memcpy_all_gather, memcpy_send_recv)
        tr.import_weights(path)
        return tr

    # ------------------------------------------------------------------ weights / checkpoints
    def init_weights(self, seed: int = 42) -> None:
        if self._pool:
            return self._pool.call("init_weights", seed)
        self.model.init_weights(seed)

    def import_weights(self, path: str) -> None:
        if self._pool:
            return self._pool.call("import_weights", str(path))
        from .utils.hf_io import import_hf_weights
        import_hf_weights(self.model, str(path))

    def export_model(self, path: str) -> None:
        if self._pool:
            return self._pool.call("export_model", str(path))
        from .utils.hf_io import export_hf_model
        export_hf_model(self.model, str(path))

    def save_checkpoint(self, directory: str, step: int, extra: Optional[dict] = None) -> None:
        if self._pool:
            return self._pool.call("save_checkpoint", str(directory), step, extra)
        from .training.checkpoint import save_checkpoint
        save_checkpoint(str(directory), step, self.model, extra or {})

    def load_checkpoint(self, directory: str, step: int) -> dict:
        if self._pool:
            return self._pool.call("load_checkpoint", str(directory), step)
        from .training.checkpoint import load_checkpoint
        return load_checkpoint(str(directory), step, self.model)

    # ------------------------------------------------------------------ training
    def _local_rows(self, a: torch.Tensor) -> torch.Tensor:
        B = self.batch_size
        if a.shape[0] == B:
            return a
        if a.shape[0] == B * self.world_size:
            return a[self.rank * B:(self.rank + 1) * B]
        raise ValueError(f"expected {B} or {B * self.world_size} rows of tokens, got {a.shape[0]}")

    def step(self, inputs, targets, z_loss: float = 0.0) -> None:
        """One micro-step (forward + backward) on int32 token arrays; returns as soon as the work is queued."""
        if self._pool:
            self._pool.step(_as_tensor(inputs), _as_tensor(targets), z_loss)
            return
        x, y = self._local_rows(_as_tensor(inputs)), self._local_rows(_as_tensor(targets))
        if self.device.type == "cuda" and not x.is_cuda:
            if self._copy_pending:
                self._copied.synchronize()              # the previous H2D copies have left the pinned buffers
            self._in_pinned.copy_(x)
            self._tg_pinned.copy_(y)
            self.model.inputs.copy_(self._in_pinned, non_blocking=True)
            self.model.targets.copy_(self._tg_pinned, non_blocking=True)
            self._copied.record()
            self._copy_pending = True
            x = y = None
        self.model.forward(x, self._micro)
        self.model.backward(x, y, z_loss, self.grad_accum, self._micro)
        self._micro += 1

    def validate(self, inputs, targets):
        if self._pool:
            return self._pool.validate(_as_tensor(inputs), _as_tensor(targets))
        x, y = self._local_rows(_as_tensor(inputs)), self._local_rows(_as_tensor(targets))
        return self.model.validate(x, y)

    def update(self, lr: float, beta1: float = 0.9, beta2: float = 0.95, step: int = 1, weight_decay: float = 0.1,
               grad_clip: float = 1.0, eps: float = 1e-8) -> Dict[str, float]:
        """Optimizer step; blocks until the step has finished and returns {loss, loss_1k, norm, z_max, z_mean}."""
        if self._pool:
            return self._pool.call("update", lr, beta1, beta2, step, weight_decay, grad_clip, eps)
        if self._micro != self.grad_accum:
            raise RuntimeError(f"update() after {self._micro} micro-steps, expected {self.grad_accum}")
        res = self.model.update(lr, beta1, beta2, step, eps, weight_decay, grad_clip, self.grad_accum)
        self._micro = 0
        self._steps_done = getattr(self, "_steps_done", 0) + 1
        return res

    # ------------------------------------------------------------------ introspection
    def get_gradients(self, gpu_id: int = 0):
        if self._pool:
            return self._pool.call_rank(gpu_id, "get_gradients", 0)
        return self.model.get_gradients()

    def get_gpu_info(self):
        from .utils.gpu_info import GPUUtilTracker
        if self._pool:
            return self._pool.call("get_gpu_info")
        if not hasattr(self, "_tracker"):
            self._tracker = GPUUtilTracker(self.device.index or 0) if self.device.type == "cuda" else None
        return [self._tracker.update()] if self._tracker else []

    def get_allocator_info(self, gpu_id: int = 0):
        if self._pool:
            return self._pool.call_rank(gpu_id, "get_allocator_info", 0)
        from .utils.memory import allocator_report
        return allocator_report(self.model)

    def close(self) -> None:
        """Collective over the ranks: releases the peer-memory segments of the in-kernel collectives in a fixed order
        (call it on every rank, with no step in flight), and stops the worker processes of the multi-GPU front end."""
        if self._pool:
            self._pool.close()
            self._pool = None
        elif getattr(self, "model", None) is not None:
            self.model.close()
