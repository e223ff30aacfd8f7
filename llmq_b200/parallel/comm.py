"""Communication back-ends behind one small interface.

``Communicator`` is what the model, the ZeRO managers and the checkpoint code talk to.  Implementations:

* ``LocalComm``      - world size 1, every collective is the identity.
* ``TorchDistComm``  - one process per GPU, ``torch.distributed`` with NCCL over NVLink/NVSwitch (or gloo on
  CPU, which is what the multi-rank CPU tests use).  This is the library baseline path and the plumbing
  (rendez-vous, tiny scalars, host gathers) for the fused in-kernel collectives of ``parallel/fused.py``.
* ``ThreadComm``     - one thread per rank inside a single process (``parallel/threads.py``).

The reference's counterpart is NCCLCommunicator with its MPI and threads flavours (src/utilities/comm.h:39-125,
src/utilities/comm.cpp).  Collectives are asynchronous: they are ordered after the work already queued on the
calling stream and return a handle whose ``wait()`` orders the calling stream after the collective, so a
gather for layer l+1 overlaps the compute of layer l.
"""
from __future__ import annotations

import os
from typing import Any, List, Optional

import torch


class _Done:
    def wait(self):
        return None


class _WorkList:
    def __init__(self, works):
        self.works = [w for w in works if w is not None]

    def wait(self):
        for w in self.works:
            w.wait()
        self.works = []


class Communicator:
    rank: int = 0
    world: int = 1

    # ---- device collectives (async; return a handle with .wait())
    def all_gather(self, full: torch.Tensor, shard: torch.Tensor):
        raise NotImplementedError

    def reduce_scatter_avg(self, full: torch.Tensor):
        """In place: afterwards rows [r*n/w, (r+1)*n/w) of ``full`` on rank r hold the mean over ranks."""
        raise NotImplementedError

    def all_reduce(self, t: torch.Tensor, op: str = "sum"):
        raise NotImplementedError

    # ---- host collectives
    def barrier(self) -> None:
        raise NotImplementedError

    def host_all_gather(self, obj: Any) -> List[Any]:
        raise NotImplementedError

    def host_gather(self, obj: Any) -> Optional[List[Any]]:
        r = self.host_all_gather(obj)
        return r if self.rank == 0 else None

    def shutdown(self) -> None:
        pass

    # ---- helpers
    def shard_rows(self, n_rows: int):
        if n_rows % self.world:
            raise ValueError(f"cannot shard {n_rows} rows over {self.world} ranks exactly")
        per = n_rows // self.world
        return self.rank * per, (self.rank + 1) * per

    def local_shard(self, full: torch.Tensor) -> torch.Tensor:
        a, b = self.shard_rows(full.shape[0])
        return full[a:b]


class LocalComm(Communicator):
    def __init__(self):
        self.rank, self.world = 0, 1

    def all_gather(self, full, shard):
        if full.data_ptr() != shard.data_ptr():
            full.view(-1)[: shard.numel()].copy_(shard.reshape(-1))
        return _Done()

    def reduce_scatter_avg(self, full):
        return _Done()

    def all_reduce(self, t, op="sum"):
        return _Done()

    def barrier(self):
        pass

    def host_all_gather(self, obj):
        return [obj]


class TorchDistComm(Communicator):
    """torch.distributed-backed communicator (NCCL on GPUs, gloo on CPU)."""

    def __init__(self, device: Optional[torch.device] = None, timeout_s: float = 1800.0, group=None):
        import torch.distributed as dist
        import datetime

        self.dist = dist
        if not dist.is_initialized():
            backend = "nccl" if (device is not None and device.type == "cuda") else "gloo"
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            kwargs = {}
            if backend == "nccl":
                kwargs["device_id"] = device
                # NCCL is plumbing here (rendez-vous, barriers, the library-collectives mode); the in-kernel collectives map
                # their own NVSwitch multicast objects over the same GPUs.  Keep NCCL off NVLS so that two owners never bind
                # memory to multicast objects of one device at the same time (set NCCL_NVLS_ENABLE yourself to override).
                os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
            dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s), **kwargs)
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.backend = dist.get_backend(group)
        self.device = device

    def all_gather(self, full, shard):
        if self.world == 1:
            return LocalComm.all_gather(self, full, shard)
        flat = full.view(-1) if full.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2) else full.view(torch.uint8).view(-1)
        sh = shard.reshape(-1) if shard.dtype not in (torch.float8_e4m3fn, torch.float8_e5m2) else shard.view(torch.uint8).reshape(-1)
        if self.backend == "gloo":
            parts = [torch.empty_like(sh) for _ in range(self.world)]
            self.dist.all_gather(parts, sh.contiguous(), group=self.group)
            flat.copy_(torch.cat(parts))
            return _Done()
        return self.dist.all_gather_into_tensor(flat, sh, group=self.group, async_op=True)

    def reduce_scatter_avg(self, full):
        if self.world == 1:
            return _Done()
        flat = full.view(-1)
        n = flat.numel() // self.world
        out = flat[self.rank * n:(self.rank + 1) * n]
        if self.backend == "gloo":
            tmp = flat.float() if flat.dtype == torch.bfloat16 else flat.clone()
            self.dist.all_reduce(tmp, group=self.group)
            out.copy_((tmp[self.rank * n:(self.rank + 1) * n] / self.world).to(flat.dtype))
            return _Done()
        return self.dist.reduce_scatter_tensor(out, flat, op=self.dist.ReduceOp.AVG, group=self.group, async_op=True)

    def all_reduce(self, t, op="sum"):
        if self.world == 1:
            return _Done()
        d = self.dist
        if op == "avg" and self.backend == "gloo":
            d.all_reduce(t, group=self.group)
            t.div_(self.world)
            return _Done()
        rop = {"sum": d.ReduceOp.SUM, "max": d.ReduceOp.MAX, "avg": d.ReduceOp.AVG}[op]
        w = d.all_reduce(t, op=rop, group=self.group, async_op=True)
        if self.backend == "gloo":
            w.wait()
            return _Done()
        return w

    def barrier(self):
        if self.world > 1:
            if self.backend == "nccl":
                self.dist.barrier(group=self.group, device_ids=[self.device.index])
            else:
                self.dist.barrier(group=self.group)

    def host_all_gather(self, obj):
        if self.world == 1:
            return [obj]
        out = [None] * self.world
        self.dist.all_gather_object(out, obj, group=self.group)
        return out

    def shutdown(self):
        if self.dist.is_initialized():
            try:
                self.dist.destroy_process_group()
            except Exception:      # a failed peer must not turn teardown into a second error
                pass


def make_communicator(device: Optional[torch.device] = None) -> Communicator:
    """World size from the launcher environment (torchrun's RANK/WORLD_SIZE or Open MPI's OMPI_COMM_WORLD_*)."""
    if "OMPI_COMM_WORLD_SIZE" in os.environ and "WORLD_SIZE" not in os.environ:
        os.environ["WORLD_SIZE"] = os.environ["OMPI_COMM_WORLD_SIZE"]
        os.environ["RANK"] = os.environ["OMPI_COMM_WORLD_RANK"]
        os.environ.setdefault("LOCAL_RANK", os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", os.environ["RANK"]))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29511")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return LocalComm()
    return TorchDistComm(device)
