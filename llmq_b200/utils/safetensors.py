"""safetensors reading / writing and Hugging Face cache lookup, without the ``safetensors`` package.

Capabilities of the reference's SafeTensorsReader/Writer (src/utilities/safetensors.h:67-131, safetensors.cpp):
single files or ``*.index.json`` shard sets, partial reads of a tensor (a row range goes straight into device
memory through the native pinned double-buffered reader, with optional dtype conversion), and a writer where
several ranks fill disjoint byte ranges of one memory-mapped output file that becomes visible atomically
(``file.tmp`` + rename).  The hub lookup never downloads (safetensors.cpp:353-393).
"""
from __future__ import annotations

import ctypes
import json
import os
import struct
from typing import Dict, List, Optional, Tuple

import torch

from ..config import safetensors_dtype, safetensors_dtype_name
from ..ops import lib as L


def _rt():
    rt = L.runtime()
    if not getattr(rt, "_io_ready", False):
        rt.llmq_rt_map_file.restype = ctypes.c_void_p
        rt._io_ready = True
    return rt


def resolve_model_dir(name: str) -> str:
    """A directory is returned as is; otherwise ``org/name`` is looked up in the local HF hub cache
    ($HF_HOME/hub, $XDG_CACHE_HOME/huggingface/hub, ~/.cache/huggingface/hub), newest snapshot first."""
    if os.path.isdir(name):
        return name
    roots = []
    if os.environ.get("HF_HOME"):
        roots.append(os.path.join(os.environ["HF_HOME"], "hub"))
    if os.environ.get("XDG_CACHE_HOME"):
        roots.append(os.path.join(os.environ["XDG_CACHE_HOME"], "huggingface", "hub"))
    roots.append(os.path.join(os.path.expanduser("~"), ".cache", "huggingface", "hub"))
    folder = "models--" + name.replace("/", "--")
    for root in roots:
        snaps = os.path.join(root, folder, "snapshots")
        if os.path.isdir(snaps):
            cands = sorted((os.path.join(snaps, d) for d in os.listdir(snaps)), key=os.path.getmtime, reverse=True)
            for c in cands:
                if os.path.exists(os.path.join(c, "config.json")):
                    return c
    raise FileNotFoundError(f"model '{name}' is neither a directory nor in the local Hugging Face cache (nothing is downloaded)")


class TensorEntry:
    __slots__ = ("name", "dtype", "shape", "file", "begin", "end")

    def __init__(self, name, dtype, shape, file, begin, end):
        self.name, self.dtype, self.shape, self.file, self.begin, self.end = name, dtype, tuple(shape), file, begin, end

    @property
    def nbytes(self):
        return self.end - self.begin


def _read_header(path: str) -> Tuple[dict, int]:
    with open(path, "rb") as f:
        raw = f.read(8)
        if len(raw) != 8:
            raise ValueError(f"{path}: truncated safetensors file")
        (n,) = struct.unpack("<Q", raw)
        if n > (1 << 30):
            raise ValueError(f"{path}: implausible header size {n}")
        hdr = f.read(n)
        if len(hdr) != n:
            raise ValueError(f"{path}: truncated safetensors header")
    return json.loads(hdr), 8 + n


class SafeTensorsReader:
    def __init__(self, path: str):
        """``path``: a ``.safetensors`` file, a ``.index.json`` file, or a directory containing either."""
        if os.path.isdir(path):
            idx = os.path.join(path, "model.safetensors.index.json")
            path = idx if os.path.exists(idx) else os.path.join(path, "model.safetensors")
        self.entries: Dict[str, TensorEntry] = {}
        self.metadata: dict = {}
        files = [path]
        if path.endswith(".index.json"):
            with open(path) as f:
                wm = json.load(f)["weight_map"]
            base = os.path.dirname(path)
            files = sorted({os.path.join(base, v) for v in wm.values()})
        for fp in files:
            hdr, data_start = _read_header(fp)
            size = os.path.getsize(fp)
            for name, info in hdr.items():
                if name == "__metadata__":
                    self.metadata.update(info)
                    continue
                b, e = info["data_offsets"]
                if data_start + e > size:
                    raise ValueError(f"{fp}: tensor {name} extends past the end of the file (truncated?)")
                self.entries[name] = TensorEntry(name, safetensors_dtype(info["dtype"]), info["shape"], fp, data_start + b, data_start + e)

    def names(self) -> List[str]:
        return list(self.entries)

    def __contains__(self, name):
        return name in self.entries

    def read_into(self, name: str, dst: torch.Tensor, elem_offset: int = 0, allow_cast: bool = True) -> None:
        """Fills ``dst`` (contiguous, any device) with ``dst.numel()`` elements starting at ``elem_offset`` of the stored tensor."""
        e = self.entries[name]
        esz = torch.empty(0, dtype=e.dtype).element_size()
        n = dst.numel()
        total = 1
        for s in e.shape:
            total *= s
        if elem_offset + n > total:
            raise ValueError(f"read of {n} elements at {elem_offset} exceeds tensor {name} with {total} elements")
        if e.dtype == dst.dtype:
            target = dst
        elif allow_cast:
            target = torch.empty(n, dtype=e.dtype, device=dst.device)
        else:
            raise TypeError(f"tensor {name} is {e.dtype}, destination is {dst.dtype}")
        if not target.is_contiguous():
            raise ValueError("destination must be contiguous")
        stream = ctypes.c_void_p(torch.cuda.current_stream(target.device).cuda_stream) if target.is_cuda else ctypes.c_void_p(0)
        rc = _rt().llmq_rt_read_file(e.file.encode(), ctypes.c_longlong(e.begin + elem_offset * esz), ctypes.c_longlong(n * esz),
                                     ctypes.c_void_p(target.data_ptr()), int(target.is_cuda), stream)
        if rc != 0:
            raise IOError(f"reading {name} from {e.file} failed with code {rc}")
        if target is not dst:
            dst.copy_(target.view(dst.shape).to(dst.dtype))

    def read(self, name: str, device="cpu") -> torch.Tensor:
        e = self.entries[name]
        t = torch.empty(e.shape, dtype=e.dtype, device=device)
        self.read_into(name, t)
        return t


class SafeTensorsWriter:
    """register() every tensor on every rank -> prepare() -> write()/write_raw() -> finalize()."""

    def __init__(self, path: str, metadata: Optional[dict] = None):
        self.path = path
        self.tmp = path + ".tmp"
        self.metadata = {"format": "pt", "writer": "llmq_b200"}
        self.metadata.update(metadata or {})
        self._reg: List[Tuple[str, torch.dtype, tuple]] = []
        self._offsets: Dict[str, Tuple[int, int]] = {}
        self._map = None
        self._size = 0

    def register(self, name: str, dtype: torch.dtype, shape) -> None:
        self._reg.append((name, dtype, tuple(int(s) for s in shape)))

    def prepare(self, create: bool = True) -> None:
        """Lays the file out.  The rank with ``create=True`` creates and sizes ``path.tmp``; the others map it
        after a barrier of the caller's choosing."""
        hdr, off = {"__metadata__": {k: str(v) for k, v in self.metadata.items()}}, 0
        for name, dt, shape in self._reg:
            n = 1
            for s in shape:
                n *= s
            nb = n * torch.empty(0, dtype=dt).element_size()
            hdr[name] = {"dtype": safetensors_dtype_name(dt), "shape": list(shape), "data_offsets": [off, off + nb]}
            self._offsets[name] = (off, off + nb)
            off += nb
        blob = json.dumps(hdr, separators=(",", ":")).encode()
        blob += b" " * ((8 - len(blob) % 8) % 8)
        self._data_start = 8 + len(blob)
        self._size = self._data_start + off
        m = _rt().llmq_rt_map_file(self.tmp.encode(), ctypes.c_longlong(self._size), int(create))
        if not m:
            raise IOError(f"could not map {self.tmp}")
        self._map = ctypes.c_void_p(m)
        if create:
            head = struct.pack("<Q", len(blob)) + blob
            ctypes.memmove(self._map, head, len(head))

    def write_raw(self, name: str, src: torch.Tensor, byte_offset: int = 0) -> None:
        """Copies the bytes of ``src`` (device or host, contiguous) to ``byte_offset`` inside tensor ``name``."""
        b, e = self._offsets[name]
        nb = src.numel() * src.element_size()
        if byte_offset < 0 or b + byte_offset + nb > e:
            raise ValueError(f"write of {nb} bytes at {byte_offset} does not fit tensor {name}")
        src = src.contiguous()
        stream = ctypes.c_void_p(torch.cuda.current_stream(src.device).cuda_stream) if src.is_cuda else ctypes.c_void_p(0)
        rc = _rt().llmq_rt_write_to_map(self._map, ctypes.c_longlong(self._data_start + b + byte_offset), ctypes.c_void_p(src.data_ptr()),
                                        ctypes.c_longlong(nb), int(src.is_cuda), stream)
        if rc != 0:
            raise IOError(f"writing {name} failed with code {rc}")

    def write(self, name: str, src: torch.Tensor) -> None:
        self.write_raw(name, src, 0)

    def finalize(self, rename: bool = True) -> None:
        """Unmaps; the rank with ``rename=True`` makes the file visible under its final name (after a barrier)."""
        if self._map is not None:
            rc = _rt().llmq_rt_unmap_file(self._map, ctypes.c_longlong(self._size), 1)
            self._map = None
            if rc != 0:
                raise IOError(f"unmapping {self.tmp} failed with code {rc}")
        if rename:
            os.replace(self.tmp, self.path)


def save_file(tensors: Dict[str, torch.Tensor], path: str, metadata: Optional[dict] = None) -> None:
    w = SafeTensorsWriter(path, metadata)
    for n, t in tensors.items():
        w.register(n, t.dtype, t.shape)
    w.prepare(True)
    for n, t in tensors.items():
        w.write(n, t)
    w.finalize(True)


def load_file(path: str, device="cpu") -> Dict[str, torch.Tensor]:
    r = SafeTensorsReader(path)
    return {n: r.read(n, device) for n in r.names()}
