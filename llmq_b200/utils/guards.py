"""Guard words around device buffers: the stand-in for a memory checker in the GPU tests.

A kernel that writes outside its output does not fault on a busy allocator: it silently changes a neighbouring tensor.
``GuardedAllocator.empty`` returns a tensor that sits between two guard zones filled with a fixed byte pattern;
``check()`` reports every zone whose pattern changed, with the name of the buffer and the offset of the first damaged
byte.  ``guard_torch_allocations()`` patches ``torch.zeros`` / ``torch.empty`` / ``torch.zeros_like`` / ``torch.empty_like``
/ ``torch.full`` for CUDA tensors inside a ``with`` block, so an existing test gets the check without being rewritten
(tests/conftest.py does that for every GPU kernel test).  The reference has nothing like it (its kernels are checked with
compute-sanitizer by hand); here every kernel test runs with the guards on.
"""
from __future__ import annotations

import contextlib
from typing import List, Tuple

import torch

GUARD_BYTES = 4096
PATTERN = 0xA5
# the allocator itself must keep using the real factories while they are patched
_torch_full, _torch_empty = torch.full, torch.empty


class GuardedAllocator:
    def __init__(self, device="cuda", guard_bytes: int = GUARD_BYTES):
        self.device = torch.device(device)
        self.guard = int(guard_bytes)
        self._live: List[Tuple[str, torch.Tensor, int]] = []          # (name, raw buffer, payload bytes)

    def empty(self, shape, dtype: torch.dtype, name: str = "", fill=None) -> torch.Tensor:
        if isinstance(shape, int):
            shape = (shape,)
        n = 1
        for s in shape:
            n *= int(s)
        es = _torch_empty(0, dtype=dtype).element_size()
        payload = n * es
        padded = (payload + 255) // 256 * 256                          # keeps the payload's natural alignment behind the guard
        raw = _torch_full((self.guard + padded + self.guard,), PATTERN, dtype=torch.uint8, device=self.device)
        view = raw[self.guard:self.guard + payload].view(dtype).view(*shape)
        if fill is not None:
            view.fill_(fill)
        self._live.append((name or f"buffer{len(self._live)}", raw, payload))
        return view

    def check(self) -> List[str]:
        """Messages for all damaged guard zones (empty list = every write stayed inside its buffer); synchronises."""
        problems = []
        for name, raw, payload in self._live:
            front = raw[:self.guard]
            back = raw[self.guard + payload:]
            for where, zone in (("before", front), ("after", back)):
                bad = (zone != PATTERN).nonzero()
                if bad.numel():
                    first = int(bad[0].item())
                    off = first - self.guard if where == "before" else first
                    problems.append(f"{name} ({tuple(raw.shape)} raw bytes, payload {payload}): guard {where} the buffer damaged, "
                                    f"{bad.numel()} bytes, first at offset {off:+d} relative to the {'start' if where == 'before' else 'end'}")
        return problems

    def release(self) -> None:
        self._live.clear()


@contextlib.contextmanager
def guard_torch_allocations(device="cuda", guard_bytes: int = GUARD_BYTES):
    """Every CUDA tensor created through the patched torch factories inside the block sits between guard zones; on exit
    (and on demand through the yielded allocator's ``check``) damaged zones raise an ``AssertionError``."""
    alloc = GuardedAllocator(device, guard_bytes)
    orig = {n: getattr(torch, n) for n in ("zeros", "empty", "zeros_like", "empty_like", "full", "ones")}

    def _is_cuda(dev) -> bool:
        return dev is not None and torch.device(dev).type == "cuda"

    def _shape(args):
        if len(args) == 1 and isinstance(args[0], (tuple, list, torch.Size)):
            return tuple(args[0])
        return tuple(int(a) for a in args)

    def make(fill):
        def factory(*args, dtype=None, device=None, **kw):
            if not _is_cuda(device) or kw.get("pin_memory") or kw.get("requires_grad") or kw.get("out") is not None:
                name = {0.0: "zeros", 1.0: "ones", None: "empty"}[fill]
                return orig[name](*args, dtype=dtype, device=device, **kw)
            return alloc.empty(_shape(args), dtype or torch.get_default_dtype(), fill=fill)
        return factory

    def full(size, fill_value, *, dtype=None, device=None, **kw):
        if not _is_cuda(device):
            return orig["full"](size, fill_value, dtype=dtype, device=device, **kw)
        dt = dtype or (torch.get_default_dtype() if isinstance(fill_value, float) else torch.int64)
        return alloc.empty(tuple(size) if not isinstance(size, int) else (size,), dt, fill=fill_value)

    def make_like(fill):
        def factory(t, *, dtype=None, device=None, **kw):
            dev = device if device is not None else t.device
            if not _is_cuda(dev) or kw.get("memory_format") not in (None, torch.preserve_format, torch.contiguous_format):
                return orig["zeros_like" if fill == 0.0 else "empty_like"](t, dtype=dtype, device=device, **kw)
            return alloc.empty(tuple(t.shape), dtype or t.dtype, fill=fill)
        return factory

    patched = {"zeros": make(0.0), "ones": make(1.0), "empty": make(None), "full": full,
               "zeros_like": make_like(0.0), "empty_like": make_like(None)}
    for n, f in patched.items():
        setattr(torch, n, f)
    try:
        yield alloc
    finally:
        for n, f in orig.items():
            setattr(torch, n, f)
    problems = alloc.check()
    alloc.release()
    assert not problems, "out-of-bounds device writes:\n  " + "\n  ".join(problems)
