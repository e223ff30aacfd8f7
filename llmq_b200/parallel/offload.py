"""Host-offload engine: pinned host memory <-> device staging with double buffers on side streams.

One pattern serves master weights, Adam moments and gradient shards during ``update`` and the per-layer residual
stream between forward and backward (reference: llama_weights.cpp:357-432, adamw_optimizer.cpp:36-159,
llama_run_state.cpp:196-260): ``fetch`` = wait until the staging buffer is free -> ``cudaMemcpyAsync`` H2D on the
fetch stream -> event; the consumer stream waits on that event; ``store`` = the store stream waits for the
producer -> D2H -> "buffer free" event.  Item i+1 is fetched while item i is being processed.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from ..utils import nvtx


class Stager:
    """Double-buffered staging for a sequence of work items (parity = item index & 1)."""

    def __init__(self, device: torch.device, zero_copy: bool = False):
        self.device = device
        self.enabled = device.type == "cuda"
        # --use-zero-copy: no staging at all, the kernels read and write the pinned host tensors through their device mapping
        # (the reference's alternative to double-buffered cudaMemcpy for offloaded optimizer state, adamw_optimizer.cpp:36-159)
        self.zero_copy = zero_copy and self.enabled
        self._alias: Dict[int, torch.Tensor] = {}
        if self.enabled:
            self.h2d = torch.cuda.Stream(device)
            self.d2h = torch.cuda.Stream(device)
        self.bufs: Dict[Tuple[str, int], torch.Tensor] = {}
        self.free: Dict[Tuple[str, int], "torch.cuda.Event"] = {}
        self.consumed: Dict[int, "torch.cuda.Event"] = {}

    def _buf(self, key, like: torch.Tensor) -> torch.Tensor:
        b = self.bufs.get(key)
        n = like.numel()
        if b is None or b.dtype != like.dtype or b.numel() < n:
            b = torch.empty(n, dtype=like.dtype, device=self.device)
            self.bufs[key] = b
        return b[:n].view(like.shape)

    def fetch(self, t: torch.Tensor, kind: str, parity: int):
        """-> (device tensor, event or None).  Device-resident tensors pass through untouched."""
        if not self.enabled or t.device.type == self.device.type:
            return t, None
        if self.zero_copy:
            a = self._alias.get(t.data_ptr())
            if a is None or a.shape != t.shape or a.dtype != t.dtype:
                from ..utils.memory import device_alias
                a = self._alias[t.data_ptr()] = device_alias(t, self.device)
            return a, None
        key = (kind, parity)
        buf = self._buf(key, t)
        with nvtx.range("offload fetch", self.device), torch.cuda.stream(self.h2d):
            if key in self.free:
                self.h2d.wait_event(self.free[key])         # the previous content has been written back
            if parity in self.consumed:
                self.h2d.wait_event(self.consumed[parity])  # ... and the kernel that read it has finished
            buf.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.h2d)
        return buf, ev

    def mark_consumed(self, parity: int) -> None:
        if not self.enabled:
            return
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        self.consumed[parity] = ev

    def store(self, staged: torch.Tensor, host: torch.Tensor, kind: str, parity: int) -> None:
        """Writes ``staged`` (produced on the current stream) back to pinned ``host`` on the store stream."""
        if not self.enabled or staged is host or staged.data_ptr() == host.data_ptr():
            return
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        with nvtx.range("offload store", self.device), torch.cuda.stream(self.d2h):
            self.d2h.wait_event(ready)
            host.copy_(staged, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.d2h)
        self.free[(kind, parity)] = ev

    def finish(self) -> None:
        """The current stream waits for all outstanding write-backs."""
        if self.enabled:
            torch.cuda.current_stream(self.device).wait_stream(self.d2h)


class ResidualStore:
    """The residual stream entering every layer (needed again in backward).

    Without offload: one device tensor per layer.  With ``offload_residual``: two device buffers plus one pinned
    host copy per layer; forward streams each finished layer input to the host, backward fetches layer l-1 while
    layer l is being processed, so device activation memory no longer grows with depth.
    """

    def __init__(self, n: int, shape, dtype, device: torch.device, offload: bool):
        self.n, self.device = n, device
        self.offload = offload and device.type == "cuda"
        if not self.offload:
            self.dev = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(n)]
            return
        self.dev = [torch.zeros(shape, dtype=dtype, device=device) for _ in range(3)]
        self.host = [torch.zeros(shape, dtype=dtype, pin_memory=True) for _ in range(n)]
        self.side = torch.cuda.Stream(device)
        self.stored: List[Optional[torch.cuda.Event]] = [None] * n      # D2H of slot i finished
        self.fetched: List[Optional[torch.cuda.Event]] = [None] * n     # H2D of slot i finished
        self.holds = [-1, -1, -1]

    # ---- forward
    def write_target(self, i: int) -> torch.Tensor:
        """Buffer into which the current stream is about to write slot i."""
        if not self.offload:
            return self.dev[i]
        b = i % 3
        old = self.holds[b]
        if old >= 0 and self.stored[old] is not None:
            torch.cuda.current_stream(self.device).wait_event(self.stored[old])    # its copy to the host is complete
        self.holds[b] = i
        return self.dev[b]

    def written(self, i: int) -> None:
        """Slot i is final on the current stream: start its copy to the host."""
        if not self.offload:
            return
        ready = torch.cuda.Event()
        ready.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self.side):
            self.side.wait_event(ready)
            self.host[i].copy_(self.dev[i % 3], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.side)
        self.stored[i] = ev

    def current(self, i: int) -> torch.Tensor:
        """Slot i while it is still resident from the forward pass (read by the layer that consumes it)."""
        return self.dev[i] if not self.offload else self.dev[i % 3]

    # ---- backward
    def prefetch(self, i: int) -> None:
        if not self.offload or i < 0 or i >= self.n:
            return
        b = i % 3
        if self.holds[b] == i:
            return
        done = torch.cuda.Event()
        done.record(torch.cuda.current_stream(self.device))             # readers of the buffer's old content
        with torch.cuda.stream(self.side):
            self.side.wait_event(done)
            if self.stored[i] is not None:
                self.side.wait_event(self.stored[i])
            self.dev[b].copy_(self.host[i], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.side)
        self.fetched[i] = ev
        self.holds[b] = i

    def get(self, i: int) -> torch.Tensor:
        """Slot i for the backward pass (waits for its fetch when it had been evicted)."""
        if not self.offload:
            return self.dev[i]
        if self.holds[i % 3] != i:
            self.prefetch(i)
        if self.fetched[i] is not None:
            torch.cuda.current_stream(self.device).wait_event(self.fetched[i])
            self.fetched[i] = None
        return self.dev[i % 3]
