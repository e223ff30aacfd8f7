"""Worker pool behind ``LLMQTrainer(ngpu > 1)`` in a single Python process.

The reference's MultiGPUPyTrainer keeps one worker thread per GPU, each spinning on a mailbox of closures, and lets
Python see one object (src/binding/py_train.cpp:19-46,97-118,189-256).  Here every GPU gets a worker *process*
(own interpreter, own CUDA context, NCCL rank), driven through a pipe: ``step`` splits the ``(ngpu*B, T)`` token
arrays by rank and returns once every worker has queued its forward/backward; ``update`` and the other calls
return rank 0's result.  A worker that raises sends the exception back and the pool re-raises it in the caller;
the remaining workers are then shut down instead of being left to wait in a collective.
"""
from __future__ import annotations

import os
import socket
import traceback
from typing import Any, List

import torch
import torch.multiprocessing as mp


def _worker(rank: int, world: int, port: int, conn, cfg, opts, B: int, T: int, GA: int, use_cuda: bool):
    try:
        os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        from ..api import LLMQTrainer
        tr = LLMQTrainer(ngpu=world, config=cfg, options=opts, batch_size=B, seq_len=T, grad_accum=GA,
                         device=None if use_cuda else "cpu")
        conn.send(("ready", None))
    except BaseException as e:                                   # noqa: BLE001
        conn.send(("error", f"{e!r}\n{traceback.format_exc()}"))
        return
    while True:
        try:
            msg = conn.recv()
        except EOFError:
            break
        name, args = msg
        if name == "close":
            try:                                                 # all workers got "close": an orderly, collective release
                tr.close()
            except Exception:
                pass
            break
        try:
            if name == "get_gradients":
                res = {k: v.float().cpu() for k, v in tr.get_gradients().items()}
            elif name == "get_gpu_info":
                res = [i.to_dict() for i in tr.get_gpu_info()]
            else:
                res = getattr(tr, name)(*args)
            conn.send(("ok", res))
        except BaseException as e:                               # noqa: BLE001
            conn.send(("error", f"{e!r}\n{traceback.format_exc()}"))
            break
    try:
        tr.comm.shutdown()
    except Exception:
        pass


class WorkerPool:
    def __init__(self, ngpu: int, cfg, opts, B: int, T: int, GA: int, use_cuda: bool = None):
        self.n, self.B = ngpu, B
        use_cuda = torch.cuda.is_available() if use_cuda is None else use_cuda
        ctx = mp.get_context("spawn")
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            port = s.getsockname()[1]
        self.conns, self.procs = [], []
        for r in range(ngpu):
            parent, child = ctx.Pipe()
            p = ctx.Process(target=_worker, args=(r, ngpu, port, child, cfg, opts, B, T, GA, use_cuda), daemon=True)
            p.start()
            self.conns.append(parent)
            self.procs.append(p)
        self._collect()

    def _collect(self) -> List[Any]:
        out, err = [], None
        for r, c in enumerate(self.conns):
            try:
                if not c.poll(1800):
                    raise TimeoutError(f"worker {r} did not answer")
                status, val = c.recv()
            except (EOFError, TimeoutError, ConnectionError) as e:
                status, val = "error", f"worker {r} died: {e!r}"
            if status == "error" and err is None:
                err = f"rank {r}: {val}"
            out.append(val)
        if err is not None:
            self.close()
            raise RuntimeError(err)
        return out

    def call(self, name: str, *args):
        for c in self.conns:
            c.send((name, args))
        return self._collect()[0]

    def call_rank(self, rank: int, name: str, *args):
        for c in self.conns:
            c.send((name, args))
        return self._collect()[rank]

    def step(self, inputs: torch.Tensor, targets: torch.Tensor, z_loss: float) -> None:
        B = self.B
        if inputs.shape[0] != B * self.n:
            raise ValueError(f"expected {B * self.n} rows of tokens, got {inputs.shape[0]}")
        for r, c in enumerate(self.conns):
            c.send(("step", (inputs[r * B:(r + 1) * B].clone(), targets[r * B:(r + 1) * B].clone(), z_loss)))
        self._collect()

    def validate(self, inputs: torch.Tensor, targets: torch.Tensor):
        B = self.B
        for r, c in enumerate(self.conns):
            c.send(("validate", (inputs[r * B:(r + 1) * B].clone(), targets[r * B:(r + 1) * B].clone())))
        return self._collect()[0]

    def close(self) -> None:
        for c in self.conns:
            try:
                c.send(("close", ()))
            except Exception:
                pass
        for p in self.procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
        self.conns, self.procs = [], []
