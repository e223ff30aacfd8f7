"""Memory bookkeeping: the LIFO temporary stack (native bookkeeping in ``csrc/rt/arena.cpp``) and the per-category
allocation report of a model.

``DeviceMemoryStack`` plays the role of the reference's stack (src/utilities/stack.h:12-52): one backing
tensor, 4 KiB-aligned LIFO blocks handed out as tensor views, a high-water mark, and a dry-run mode (no
backing memory) with which the real buffer is sized by replaying one step's allocation pattern.
``allocator_report`` groups what a model holds by the categories of the reference's memory report
(src/utilities/allocator.cpp:211-240).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch

from ..ops import lib as L


def _rt():
    rt = L.runtime()
    if not getattr(rt, "_stack_ready", False):
        rt.llmq_stack_create.restype = ctypes.c_void_p
        for f in ("llmq_stack_alloc", "llmq_stack_used", "llmq_stack_high_water", "llmq_stack_capacity"):
            getattr(rt, f).restype = ctypes.c_longlong
        rt.llmq_stack_error.restype = ctypes.c_char_p
        rt._stack_ready = True
    return rt


class DeviceMemoryStack:
    def __init__(self, capacity_bytes: int = 0, device="cpu", dry_run: bool = False):
        self.dry_run = dry_run
        self.device = torch.device(device)
        self._h = ctypes.c_void_p(_rt().llmq_stack_create(ctypes.c_longlong(capacity_bytes), int(dry_run)))
        self.backing = None if dry_run else torch.empty(max(capacity_bytes, 1), dtype=torch.uint8, device=self.device)
        self._offsets: List[int] = []

    def __del__(self):
        h = getattr(self, "_h", None)
        if h:
            try:
                _rt().llmq_stack_destroy(h)
            except Exception:
                pass

    def allocate(self, shape, dtype: torch.dtype, name: str = "") -> Optional[torch.Tensor]:
        """Returns a view of the backing buffer (``None`` in dry-run mode, where only sizes are recorded)."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = n * torch.empty(0, dtype=dtype).element_size()
        off = _rt().llmq_stack_alloc(self._h, ctypes.c_longlong(nbytes), name.encode())
        if off < 0:
            raise MemoryError(_rt().llmq_stack_error(self._h).decode())
        self._offsets.append(off)
        if self.dry_run:
            return None
        return self.backing[off:off + nbytes].view(dtype).view(*shape)

    def free(self, tensor: Optional[torch.Tensor] = None) -> None:
        """Frees the most recent block; passing the tensor checks that it really is the top of the stack."""
        if not self._offsets:
            raise RuntimeError("free on an empty stack")
        off = self._offsets[-1]
        if tensor is not None and not self.dry_run:
            t_off = tensor.data_ptr() - self.backing.data_ptr()
            if t_off != off:
                raise RuntimeError("stack blocks must be freed in reverse order of allocation")
        if _rt().llmq_stack_free(self._h, ctypes.c_longlong(off)) != 0:
            raise RuntimeError(_rt().llmq_stack_error(self._h).decode())
        self._offsets.pop()

    @property
    def used(self) -> int:
        return int(_rt().llmq_stack_used(self._h))

    @property
    def high_water(self) -> int:
        return int(_rt().llmq_stack_high_water(self._h))

    @property
    def capacity(self) -> int:
        return int(_rt().llmq_stack_capacity(self._h))

    def high_water_breakdown(self) -> Dict[str, int]:
        buf = ctypes.create_string_buffer(1 << 16)
        n = _rt().llmq_stack_high_water_report(self._h, buf, len(buf))
        out: Dict[str, int] = {}
        if n > 0:
            for item in buf.value.decode().split(";"):
                if item:
                    k, v = item.rsplit(":", 1)
                    out[k] = out.get(k, 0) + int(v)
        return out


def host_tensor(shape, dtype: torch.dtype, write_combined: bool = False) -> torch.Tensor:
    """A zero-filled CPU tensor in page-locked host memory that is mapped into the device address space (offloaded
    state).  ``write_combined`` asks for write-combined pages (``--write-combined``): fast for the device to read over
    PCIe and for the CPU to write, slow for the CPU to read - fine for state that only the GPU consumes.  Falls back to
    torch's pinned allocator when the runtime library cannot allocate (no CUDA device)."""
    n = 1
    for s_ in shape:
        n *= int(s_)
    nbytes = n * torch.empty(0, dtype=dtype).element_size()
    ptr = None
    if nbytes > 0 and torch.cuda.is_available():
        rt = L.runtime()
        rt.llmq_host_alloc.restype = ctypes.c_void_p
        ptr = rt.llmq_host_alloc(ctypes.c_longlong(nbytes), int(write_combined))
    if not ptr:
        return torch.zeros(shape, dtype=dtype, pin_memory=torch.cuda.is_available())
    buf = (ctypes.c_uint8 * nbytes).from_address(ptr)
    ctypes.memset(ptr, 0, nbytes)
    t = torch.frombuffer(buf, dtype=torch.uint8).view(dtype).view(*shape)
    import weakref
    weakref.finalize(buf, rt.llmq_host_free, ctypes.c_void_p(ptr))      # the tensor keeps `buf` alive; free when both are gone
    return t


class _CudaView:
    """Object with the CUDA array interface over an address range: lets torch build a device tensor on existing memory."""

    def __init__(self, ptr: int, shape, typestr: str):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3, "strides": None}


def device_alias(t: torch.Tensor, device: torch.device) -> torch.Tensor:
    """A CUDA tensor over the memory of a page-locked, device-mapped host tensor (zero copy): kernels read and write the
    host memory over the bus.  Under unified addressing the device pointer of mapped pinned memory equals the host pointer."""
    assert t.device.type == "cpu" and t.is_contiguous()
    raw = torch.as_tensor(_CudaView(t.data_ptr(), (t.numel() * t.element_size(),), "|u1"), device=device)
    return raw.view(t.dtype).view(t.shape)


def _nbytes(t) -> int:
    return t.numel() * t.element_size()


def _add(report, category: str, t: torch.Tensor, seen: set) -> None:
    key = (t.untyped_storage().data_ptr(), t.device.type)
    if key in seen or t.numel() == 0:
        return
    seen.add(key)
    kind = "device" if t.device.type == "cuda" else ("pinned" if t.is_pinned() else "host")
    report.setdefault(category, {"device": 0, "pinned": 0, "host": 0})[kind] += t.untyped_storage().nbytes()


def allocator_report(model) -> Dict[str, Dict[str, int]]:
    """Bytes held by ``model`` per category {Weights, Master, Quants, Adam M, Adam V, Gradients, Activations, Stack}."""
    rep: Dict[str, Dict[str, int]] = {}
    seen: set = set()
    w = model.weights
    for b in w.bufs:
        for t in b.t.values():
            _add(rep, "Weights", t, seen)
    for t in w.nb_work.values():
        _add(rep, "Weights", t, seen)
    for d in w.master_blocks:
        for t in d.values():
            _add(rep, "Master", t, seen)
    for t in w.master_nb.values():
        _add(rep, "Master", t, seen)
    if w.quant_shards:
        for d in w.quant_shards:
            for t in d.values():
                _add(rep, "Quants", t, seen)
    for t in model.opt_state.m.values():
        _add(rep, "Adam M", t, seen)
    for t in model.opt_state.m_scales.values():
        _add(rep, "Adam M", t, seen)
    for t in model.opt_state.v.values():
        _add(rep, "Adam V", t, seen)
    g = model.grads
    for coll in (getattr(g, "full", []), getattr(g, "bufs", []), getattr(g, "shards", [])):
        for d in coll:
            for t in d.values():
                _add(rep, "Gradients", t, seen)
    for t in g.nb_full.values():
        _add(rep, "Gradients", t, seen)
    for v in vars(model.acts).values():
        if hasattr(v, "dev"):                                   # ResidualStore
            v = list(v.dev) + list(getattr(v, "host", []))
        for t in (v if isinstance(v, list) else [v]):
            if isinstance(t, torch.Tensor):
                _add(rep, "Activations", t, seen)
    for t in (model.lnf, model.rstd_f, model.losses, model.lse_tok, model.stats):
        _add(rep, "Activations", t, seen)
    for t in vars(model.tmp).values():
        if isinstance(t, torch.Tensor):
            _add(rep, "Stack", t, seen)
    if getattr(model, "stack_report", None):
        rep["_stack"] = dict(model.stack_report)             # dry-run sizing of the temporaries' stack: capacity, high-water mark, who was live
    if model.device.type == "cuda":
        free, total = torch.cuda.mem_get_info(model.device)
        rep["_device"] = {"free": free, "total": total, "reserved": torch.cuda.memory_reserved(model.device)}
    return rep


def large_tensors(model, min_mib: float):
    """[(name, shape, MiB, device | pinned | host)] of the model's weight / optimizer / gradient / activation tensors
    of at least ``min_mib`` MiB (``--debug-log-allocations``), largest first."""
    seen, out = set(), []

    def add(name, t):
        if not isinstance(t, torch.Tensor) or t.numel() == 0:
            return
        key = t.untyped_storage().data_ptr()
        mib = t.untyped_storage().nbytes() / 2**20
        if key in seen or mib < min_mib:
            return
        seen.add(key)
        where = "device" if t.device.type == "cuda" else ("pinned" if t.is_pinned() else "host")
        out.append((name, tuple(t.shape), mib, where))

    w = model.weights
    for i, b in enumerate(w.bufs):
        for n, t in b.t.items():
            add(f"work[{i}].{n}", t)
    for l, d in enumerate(w.master_blocks):
        for n, t in d.items():
            add(f"master[{l}].{n}", t)
    for n, t in w.master_nb.items():
        add(f"master.{n}", t)
    for n, t in model.opt_state.m.items():
        add(f"adam_m.{n}", t)
    for n, t in model.opt_state.v.items():
        add(f"adam_v.{n}", t)
    g = model.grads
    for coll_name in ("full", "bufs", "shards"):
        for l, d in enumerate(getattr(g, coll_name, [])):
            for n, t in d.items():
                add(f"grad_{coll_name}[{l}].{n}", t)
    for n, t in g.nb_full.items():
        add(f"grad.{n}", t)
    for n, v in vars(model.acts).items():
        if hasattr(v, "dev"):
            v = list(v.dev) + list(getattr(v, "host", []))
        for i, t in enumerate(v if isinstance(v, list) else [v]):
            add(f"act.{n}[{i}]", t)
    for n, t in vars(model.tmp).items():
        add(f"tmp.{n}", t)
    return sorted(out, key=lambda e: -e[2])
