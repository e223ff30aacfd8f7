"""Token-file data loading: Python face of the native loader (``csrc/rt/dataloader.cpp``), a writer for the
``BIN.TOK`` format and a uniform-random synthetic generator.

API follows the reference's binding (src/binding/binding.cpp:330-353): ``DataLoader(file_list, chunk_size, seed)``,
``load_batch(inputs, targets)``, ``has_next(n)``, ``advance_epoch()``, ``set_state(...)``, ``epoch()``,
``progress()`` and the read-only properties.
"""
from __future__ import annotations

import ctypes
import glob as _glob
from typing import List, Optional, Sequence, Union

import numpy as np
import torch

from ..ops import lib as L

HEADER_BYTES = 1024
MAGIC = b"BIN.TOK\n"


def _rt():
    rt = L.runtime()
    if not getattr(rt, "_dl_ready", False):
        rt.llmq_dl_create.restype = ctypes.c_void_p
        rt.llmq_dl_error.restype = ctypes.c_char_p
        rt.llmq_dl_current_file.restype = ctypes.c_char_p
        rt.llmq_dl_progress.restype = ctypes.c_double
        rt._dl_ready = True
    return rt


def match_files(pattern: Union[str, Sequence[str]]) -> List[str]:
    """Expands a glob pattern (or passes a list through), sorted; raises if nothing matches."""
    if not isinstance(pattern, str):
        return list(pattern)
    files = sorted(_glob.glob(pattern))
    if not files:
        raise FileNotFoundError(f"No files found with pattern '{pattern}'")
    return files


class DataLoader:
    def __init__(self, file_list: Union[str, Sequence[str]], chunk_size: int, seed: int = 42, rank: int = 0, world_size: int = 1):
        self.files = match_files(file_list)
        self.seq_len = int(chunk_size)
        self.rank, self.world_size = rank, world_size
        rt = _rt()
        arr = (ctypes.c_char_p * len(self.files))(*[f.encode() for f in self.files])
        err = ctypes.c_char_p()
        self._h = rt.llmq_dl_create(arr, len(self.files), self.seq_len, rank, world_size, ctypes.c_ulonglong(seed), ctypes.byref(err))
        if not self._h:
            raise RuntimeError((err.value or b"could not create data loader").decode())
        self._h = ctypes.c_void_p(self._h)

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _rt().llmq_dl_destroy(h)
            except Exception:
                pass
            self._h = None

    # ---- loading
    def load_batch(self, inputs, targets) -> None:
        """Fills int32 arrays / CPU tensors of shape (batch, seq_len) (any shape with batch*seq_len elements)."""
        xi, xt = _as_int32(inputs), _as_int32(targets)
        n = xi.size if isinstance(xi, np.ndarray) else xi.numel()
        if n % self.seq_len:
            raise ValueError(f"batch of {n} tokens is not a multiple of the sequence length {self.seq_len}")
        rc = _rt().llmq_dl_load_batch(self._h, _addr(xi), _addr(xt), n // self.seq_len)
        if rc != 0:
            raise RuntimeError(_rt().llmq_dl_error(self._h).decode())

    def has_next(self, n: int = 1) -> bool:
        return bool(_rt().llmq_dl_has_next(self._h, n))

    def advance_epoch(self) -> None:
        _rt().llmq_dl_advance_epoch(self._h)

    # ---- state
    def _state(self):
        out = (ctypes.c_longlong * 8)()
        _rt().llmq_dl_get_state(self._h, out)
        return list(out)

    def set_state(self, seed: int, epoch: int, file_index: int, chunk_index: int) -> None:
        _rt().llmq_dl_set_state(self._h, ctypes.c_ulonglong(seed), epoch, file_index, ctypes.c_longlong(chunk_index))

    def get_state(self) -> dict:
        s = self._state()
        return {"seed": s[0], "epoch": s[1], "file_index": s[2], "chunk_index": s[3], "file_name": self.current_file}

    def epoch(self) -> int:
        return self._state()[1]

    def progress(self) -> float:
        return float(_rt().llmq_dl_progress(self._h))

    seed = property(lambda self: self._state()[0])
    file_index = property(lambda self: self._state()[2])
    chunk_index = property(lambda self: self._state()[3])
    num_tokens = property(lambda self: self._state()[4])
    num_chunks = property(lambda self: self._state()[5])
    vocab_size = property(lambda self: self._state()[6])
    num_files = property(lambda self: self._state()[7])
    current_file = property(lambda self: _rt().llmq_dl_current_file(self._h).decode())


def _as_int32(a):
    if isinstance(a, torch.Tensor):
        if a.dtype != torch.int32 or a.is_cuda or not a.is_contiguous():
            raise TypeError("expected a contiguous int32 CPU tensor")
        return a
    a = np.asarray(a)
    if a.dtype != np.int32 or not a.flags.c_contiguous:
        raise TypeError("expected a C-contiguous int32 array")
    return a


def _addr(a):
    return ctypes.c_void_p(a.data_ptr() if isinstance(a, torch.Tensor) else a.ctypes.data)


class TokenFileWriter:
    """Writes a version-2 ``BIN.TOK`` file; optional per-token training mask (1 = target is trained on)."""

    def __init__(self, file_name: str, vocab_size: int, masking: bool = False):
        self.file_name, self.vocab_size, self.masking = file_name, vocab_size, masking
        self.n_tokens = 0
        self._masks: List[np.ndarray] = []

    def __enter__(self):
        self._f = open(self.file_name, "wb")
        self._f.write(b"\0" * HEADER_BYTES)
        return self

    def add_document(self, tokens, mask: Optional[np.ndarray] = None) -> None:
        tokens = np.asarray(tokens, dtype=np.int32)
        self._f.write(tokens.tobytes())
        self.n_tokens += len(tokens)
        if self.masking:
            m = np.ones(len(tokens), dtype=bool) if mask is None else np.asarray(mask).astype(bool)
            if len(m) != len(tokens):
                raise ValueError("mask and tokens differ in length")
            self._masks.append(m)

    def __exit__(self, exc_type, exc, tb):
        if self.masking and exc_type is None:
            bits = np.concatenate(self._masks) if self._masks else np.zeros(0, dtype=bool)
            self._f.write(np.packbits(bits, bitorder="little").tobytes())
        self._f.seek(0)
        self._f.write(MAGIC)
        self._f.write(np.array([2, 4, self.n_tokens, self.vocab_size, int(self.masking)], dtype=np.int32).tobytes())
        self._f.close()


def write_synthetic_token_file(file_name: str, n_tokens: int, vocab_size: int, seed: int = 0) -> None:
    """Uniform-random token ids, the data used for benchmarks and tests (no dataset download needed)."""
    rng = np.random.default_rng(seed)
    with TokenFileWriter(file_name, vocab_size) as w:
        left = n_tokens
        while left > 0:
            n = min(left, 1 << 22)
            w.add_document(rng.integers(0, vocab_size, size=n, dtype=np.int32))
            left -= n
