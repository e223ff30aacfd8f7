"""One rank per thread inside a single process, with copy-engine collectives.

This is the multi-thread launch mode of the reference (NCCLCommunicatorThreads, src/utilities/comm.cpp:353-662) and at
the same time its ``--memcpy-all-gather`` / ``--memcpy-send-recv`` / ``--all-to-all-reduce`` algorithms: ranks
publish their tensors in a shared table and pull the peers' slices with plain device-to-device copies, which
run on the copy engines and take no SMs (comm.cpp:500-549).  In a shared address space no IPC handles are
needed; the exchange of pointers is an exchange of Python references.

* all-gather: every rank copies each peer's shard into its own full buffer.
* reduce-scatter (mean): every rank pulls the peers' slices *of its own shard range* and reduces them locally in
  fp32 - the "destructive all-to-all + local reduce" of the reference, without the staging slots.
* exceptions raised in one rank thread break the shared barrier, so the other ranks fail fast instead of
  waiting forever, and the launcher re-raises the first error (comm.cpp:426-494).

Python threads share the interpreter lock, so this mode is about capability (and CPU tests), not about peak
throughput with many GPUs; the process-per-GPU mode is the fast one.
"""
from __future__ import annotations

import threading
from typing import Any, Callable, List, Optional

import torch

from .comm import Communicator, _Done


class _Shared:
    def __init__(self, world: int, timeout: float):
        self.world = world
        self.barrier = threading.Barrier(world, timeout=timeout)
        self.table: List[Any] = [None] * world
        self.errors: List[Optional[BaseException]] = [None] * world


_tls = threading.local()


def current_thread_comm() -> Optional["ThreadComm"]:
    """The communicator of the calling rank thread (None outside ``run_in_threads``)."""
    return getattr(_tls, "comm", None)


class ThreadComm(Communicator):
    def __init__(self, rank: int, shared: _Shared, device: Optional[torch.device] = None):
        self.rank, self.world, self.shared, self.device = rank, shared.world, shared, device

    # ---- host collectives
    def barrier(self) -> None:
        try:
            self.shared.barrier.wait()
        except threading.BrokenBarrierError:
            raise RuntimeError(f"rank {self.rank}: a peer rank failed or timed out") from None

    def host_all_gather(self, obj: Any) -> List[Any]:
        self.shared.table[self.rank] = obj
        self.barrier()
        out = list(self.shared.table)
        self.barrier()
        return out

    def _sync_device(self) -> None:
        if self.device is not None and self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()

    # ---- device collectives (synchronous with respect to the host; copies are device-to-device)
    def all_gather(self, full: torch.Tensor, shard: torch.Tensor):
        if self.world == 1:
            return _Done()
        self._sync_device()                         # my shard is final before peers read it
        shards = self.host_all_gather(shard)
        flat = full.view(torch.uint8).view(-1) if full.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else full.view(-1)
        n = flat.numel() // self.world
        for r in range(self.world):
            if r == self.rank:
                continue
            src = shards[r]
            src = src.view(torch.uint8).reshape(-1) if src.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else src.reshape(-1)
            flat[r * n:(r + 1) * n].copy_(src, non_blocking=True)
        self._sync_device()
        self.barrier()                              # nobody overwrites a shard that a peer is still reading
        return _Done()

    def reduce_scatter_avg(self, full: torch.Tensor):
        if self.world == 1:
            return _Done()
        self._sync_device()
        fulls = self.host_all_gather(full)
        flat = full.view(-1)
        n = flat.numel() // self.world
        a, b = self.rank * n, (self.rank + 1) * n
        acc = flat[a:b].float()
        for r in range(self.world):
            if r != self.rank:
                acc += fulls[r].view(-1)[a:b].to(flat.device, non_blocking=True).float()
        acc /= self.world
        self._sync_device()
        self.barrier()                              # all peers have read my copy of their ranges
        flat[a:b].copy_(acc.to(flat.dtype))
        return _Done()

    def all_reduce(self, t: torch.Tensor, op: str = "sum"):
        if self.world == 1:
            return _Done()
        self._sync_device()
        vals = self.host_all_gather(t.detach().clone())
        stack = torch.stack([v.to(t.device).float() for v in vals])
        res = {"sum": stack.sum(0), "avg": stack.mean(0), "max": stack.max(0).values}[op]
        t.copy_(res.to(t.dtype))
        return _Done()


def run_in_threads(world: int, fn: Callable[[ThreadComm], Any], devices: Optional[List[torch.device]] = None,
                   timeout: float = 600.0) -> List[Any]:
    """Runs ``fn(comm)`` on ``world`` threads (rank i drives ``devices[i]``); returns the results by rank or re-raises
    the first error of any rank."""
    shared = _Shared(world, timeout)
    results: List[Any] = [None] * world

    def body(rank: int):
        dev = devices[rank] if devices else (torch.device("cuda", rank) if torch.cuda.is_available() else torch.device("cpu"))
        comm = ThreadComm(rank, shared, dev)
        _tls.comm = comm
        try:
            if dev.type == "cuda":
                torch.cuda.set_device(dev)
            results[rank] = fn(comm)
        except BaseException as e:                  # noqa: BLE001 - propagated to the launcher below
            shared.errors[rank] = e
            shared.barrier.abort()                  # wakes every rank that waits for this one
        finally:
            _tls.comm = None

    threads = [threading.Thread(target=body, args=(r,), name=f"llmq-rank-{r}", daemon=True) for r in range(world)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    primary = [e for e in shared.errors if e is not None and "a peer rank failed" not in str(e)]
    if primary or any(shared.errors):
        raise (primary[0] if primary else next(e for e in shared.errors if e is not None))
    return results
