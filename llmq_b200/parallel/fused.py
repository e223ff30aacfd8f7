"""In-kernel collectives over NVLink peer memory: the symmetric heap and the calls into ``csrc/p2p_collectives.cu``.

``torch.distributed`` (NCCL) is used only as plumbing here: the rendez-vous that maps every rank's heap segments into
every peer (``torch.distributed._symmetric_memory``) and a host barrier at set-up.  NCCL's own NVLink-SHARP (NVLS)
algorithms are switched off by the communicator (``parallel/comm.py``), so that only this module binds device memory to
NVSwitch multicast objects, and ``close()`` releases the segments in a fixed order on all ranks.  After that all traffic is
issued by our own kernels with loads / stores on peer addresses, or with ``multimem`` loads on the NVSwitch
multicast address when the platform offers one (``LLMQ_P2P_MULTIMEM=0`` forces plain peer loads; the failure
tests use that).

A tensor that takes part in a fused collective must live in the heap (``heap.empty``): it then has the same
(segment, offset) on every rank, which is all a kernel needs besides the table of peer base pointers.
Synchronisation uses flag words in a small heap segment: ``signal(channel)`` release-stores a generation number
into word [channel][my rank] of every peer, ``wait(channel)`` spins (bounded) on the local words until every
rank's generation arrived.  A time-out is recorded in the device status word and raised by ``check_status``.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch

from ..ops import kernels as K
from ..ops import lib as L

F8 = (torch.float8_e4m3fn, torch.float8_e5m2)
SEGMENT_BYTES = 2 << 30
MAX_CHANNELS = 4096
SMALL_SLOTS_FLOATS = 4096              # per rank and per generation parity, for the small all-reduce


class _Segment:
    def __init__(self, nbytes: int, device, group):
        import torch.distributed._symmetric_memory as symm
        self.buf = symm.empty(nbytes, dtype=torch.uint8, device=device)
        self.hdl = symm.rendezvous(self.buf, group)
        self.nbytes, self.used = nbytes, 0
        ptrs = list(self.hdl.buffer_ptrs)
        self.peer_array = (ctypes.c_void_p * 8)(*(ptrs + [0] * (8 - len(ptrs))))
        mc = int(getattr(self.hdl, "multicast_ptr", 0) or 0)
        self.multicast = mc if os.environ.get("LLMQ_P2P_MULTIMEM", "1") != "0" else 0
        self.base = self.buf.data_ptr()


class SymmetricHeap:
    def __init__(self, device: torch.device, group, segment_bytes: int = SEGMENT_BYTES):
        self.device, self.group, self.segment_bytes = device, group, segment_bytes
        self.segments: List[_Segment] = []

    def empty(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """A zero-initialised tensor at the same (segment, offset) on every rank; collective over the group
        whenever a new segment has to be mapped, so all ranks must allocate in the same order."""
        n = 1
        for s in shape:
            n *= int(s)
        nbytes = (n * torch.empty(0, dtype=dtype).element_size() + 255) // 256 * 256
        seg = next((s for s in self.segments if s.used + nbytes <= s.nbytes), None)
        if seg is None:
            seg = _Segment(max(self.segment_bytes, nbytes), self.device, self.group)
            seg.buf.zero_()
            # The clearing memset runs on this rank's stream; a faster peer could already store into the new segment (its
            # first push after the allocation) and this rank's memset would then wipe that data.  So: finish the memset,
            # then meet all ranks on the host before anybody uses the segment.
            torch.cuda.synchronize(self.device)
            import torch.distributed as dist
            dist.barrier(group=self.group, device_ids=[self.device.index])
            self.segments.append(seg)
        off = seg.used
        seg.used += nbytes
        raw = seg.buf[off:off + n * torch.empty(0, dtype=dtype).element_size()]
        return raw.view(dtype).view(*shape)

    def locate(self, t: torch.Tensor) -> Tuple[_Segment, int]:
        p = t.data_ptr()
        for s in self.segments:
            if s.base <= p < s.base + s.nbytes:
                return s, p - s.base
        raise ValueError("tensor does not live in the symmetric heap")

    def contains(self, t: torch.Tensor) -> bool:
        p = t.data_ptr()
        return any(s.base <= p < s.base + s.nbytes for s in self.segments)


class FusedCollectives:
    """Per-rank object that launches the peer-memory kernels; one side stream carries gathers and reductions."""

    def __init__(self, comm, device: torch.device, wait_limit_s: float = 20.0):
        import torch.distributed as dist
        self.comm, self.device = comm, device
        self.rank, self.world = comm.rank, comm.world
        if self.world > 8:
            raise ValueError("peer-memory collectives support up to 8 ranks (one NVSwitch domain)")
        group = comm.group if comm.group is not None else dist.group.WORLD
        self.heap = SymmetricHeap(device, group)
        self.ctrl = _Segment(1 << 20, device, group)                    # flags + small all-reduce slots
        self.ctrl.buf.zero_()
        self.flag_bytes = MAX_CHANNELS * 8 * 4
        self.slots_offset = self.flag_bytes
        self.small_channel = MAX_CHANNELS - 1
        self.gen: Dict[int, int] = {}
        self.wait_limit_s = wait_limit_s
        self.stream = torch.cuda.Stream(device)
        self.sms = K.num_sms(device)
        self.status = K.status_word(device)
        self.use_multimem = self.ctrl.multicast != 0
        torch.cuda.synchronize(device)
        comm.barrier()

    def close(self) -> None:
        """Ordered teardown, collective over the ranks: every rank finishes its device work, all ranks meet on the host,
        and only then are the symmetric segments (and with them the multicast bindings) released.  Without it a rank that
        leaves early unbinds memory that a slower peer's kernel may still be reading through the multicast address."""
        if getattr(self, "_closed", False):
            return
        self._closed = True
        torch.cuda.synchronize(self.device)
        self.comm.barrier()
        self.heap.segments.clear()
        self.ctrl = None
        torch.cuda.synchronize(self.device)
        self.comm.barrier()

    # ---- flags
    def _flag_offset(self, channel: int) -> int:
        return channel * 8 * 4

    def next_gen(self, channel: int) -> int:
        g = self.gen.get(channel, 0) + 1
        self.gen[channel] = g
        return g

    def signal(self, channel: int, gen: Optional[int] = None) -> int:
        """All earlier work of the current stream is visible to a peer that sees this generation."""
        gen = self.next_gen(channel) if gen is None else gen
        L.check(L.kernels().llmq_p2p_signal(self.ctrl.peer_array, ctypes.c_longlong(self._flag_offset(channel)), self.rank, self.world,
                                            ctypes.c_uint(gen), L.stream_ptr()), "p2p_signal")
        return gen

    def wait(self, channel: int, gen: int) -> None:
        """Current stream waits until every rank signalled ``gen`` on ``channel`` (bounded; see check_status)."""
        flags = ctypes.c_void_p(self.ctrl.base + self._flag_offset(channel))
        L.check(L.kernels().llmq_p2p_wait(flags, self.world, ctypes.c_uint(gen), L.ptr(self.status), ctypes.c_double(self.wait_limit_s),
                                          L.stream_ptr()), "p2p_wait")

    # ---- data movement
    def quant_allgather(self, full: torch.Tensor, shard: torch.Tensor, absmax: Optional[torch.Tensor] = None,
                        scale_out: Optional[torch.Tensor] = None) -> None:
        """Stores this rank's shard (quantised to ``full``'s fp8 dtype with the given abs-max, or copied) into the
        shard's slot of ``full`` on every rank."""
        seg, off = self.heap.locate(full)
        quant = full.dtype in F8
        if shard.dtype != torch.bfloat16 or (not quant and full.dtype != torch.bfloat16):
            raise TypeError("fused all-gather takes bf16 shards and writes e4m3 or bf16")
        L.check(L.kernels().llmq_p2p_quant_allgather(seg.peer_array, ctypes.c_longlong(off), L.ptr(shard), ctypes.c_longlong(shard.numel()),
                                                     self.rank, self.world, L.ptr(absmax), L.ptr(scale_out), 1 if quant else 0, self.sms,
                                                     L.stream_ptr()), "p2p_quant_allgather")

    def push_allgather(self, full: torch.Tensor, shard: torch.Tensor) -> None:
        """Stores this rank's shard, which already has ``full``'s dtype (e.g. a kept e4m3 shard, on the device or in
        pinned host memory), into its slot of ``full`` on every rank: the copy form of the kernel on the raw bytes."""
        seg, off = self.heap.locate(full)
        nbytes = shard.numel() * shard.element_size()
        if shard.dtype != full.dtype or nbytes % 16 or not shard.is_contiguous():
            raise TypeError("push all-gather takes a contiguous shard of the destination's dtype, a multiple of 16 bytes")
        L.check(L.kernels().llmq_p2p_quant_allgather(seg.peer_array, ctypes.c_longlong(off), L.ptr(shard), ctypes.c_longlong(nbytes // 2),
                                                     self.rank, self.world, None, None, 0, self.sms, L.stream_ptr()), "p2p_quant_allgather")

    # ---- copy-engine forms (--memcpy-all-gather, --memcpy-send-recv + --all-to-all-reduce in process mode)
    def _memcpy(self, dst_ptr: int, src_ptr: int, nbytes: int) -> None:
        L.check(L.kernels().llmq_memcpy_d2d_async(ctypes.c_void_p(dst_ptr), ctypes.c_void_p(src_ptr), ctypes.c_longlong(nbytes),
                                                  L.stream_ptr()), "memcpy_d2d")

    def copy_allgather(self, full: torch.Tensor) -> None:
        """This rank's slot of ``full`` (already filled locally) goes into the same slot of every peer's ``full`` with
        copy-engine transfers on the current stream, no SM involved (schedule_all_gather with memcpy in the reference,
        comm.cpp:570-590)."""
        seg, off = self.heap.locate(full)
        nbytes = full.numel() * full.element_size() // self.world
        ptrs = list(seg.hdl.buffer_ptrs)
        mine = off + self.rank * nbytes
        for k in range(1, self.world):
            p = (self.rank + k) % self.world                      # every rank starts with a different peer
            self._memcpy(ptrs[p] + mine, ptrs[self.rank] + mine, nbytes)

    def copy_all_to_all(self, full: torch.Tensor, landing: torch.Tensor) -> None:
        """Slot s of ``full`` goes into slot [this rank] of rank s's ``landing`` (same shape, in the heap) for every peer s,
        with copy-engine transfers; the own slot is copied locally.  The send half of the all-to-all reduce-scatter
        (schedule_destructive_all_to_all, comm.cpp:500-549; here the landing buffer is separate, so nothing is destroyed)."""
        seg, off = self.heap.locate(full)
        lseg, loff = self.heap.locate(landing)
        nbytes = full.numel() * full.element_size() // self.world
        src_base = list(seg.hdl.buffer_ptrs)[self.rank] + off
        lptrs = list(lseg.hdl.buffer_ptrs)
        for k in range(self.world):
            s = (self.rank + k) % self.world
            self._memcpy(lptrs[s] + loff + self.rank * nbytes, src_base + s * nbytes, nbytes)

    def sum_slots(self, landing: torch.Tensor, dst: torch.Tensor, *, accumulate: bool, scale: float,
                  norm_partials: Optional[torch.Tensor] = None, seed: int = 0) -> None:
        """dst (+)= scale * sum over the ``world`` local slots of ``landing`` (the receive half of the all-to-all reduction:
        the kernel of ``rs_finish`` without a counter to wait for; callers order it after the arrival flags)."""
        zero_counter = ctypes.c_void_p(self.ctrl.base + self.RS_COUNTER_BASE + 4 * 8000)      # a word nobody increments; target 0
        L.check(L.kernels().llmq_p2p_rs_finish(L.ptr(landing), zero_counter, ctypes.c_uint(0), ctypes.c_longlong(dst.numel()), self.rank,
                                               self.world, L.ptr(dst), int(accumulate), ctypes.c_float(scale), L.ptr(norm_partials),
                                               0 if norm_partials is None else norm_partials.numel(), ctypes.c_uint(seed & 0xFFFFFFFF),
                                               L.ptr(self.status), ctypes.c_double(self.wait_limit_s), self.sms, L.stream_ptr()), "p2p_rs_finish")

    def reduce_scatter(self, full: torch.Tensor, dst: torch.Tensor, *, accumulate: bool, scale: float,
                       norm_partials: Optional[torch.Tensor] = None, seed: int = 0) -> None:
        """dst (+)= scale * sum over ranks of rows [rank*n/w, (rank+1)*n/w) of ``full`` (bf16, in the heap)."""
        seg, off = self.heap.locate(full)
        n_shard = full.numel() // self.world
        mc = ctypes.c_void_p(seg.multicast if (seg.multicast and n_shard % 8 == 0) else 0)
        L.check(L.kernels().llmq_p2p_reduce_scatter(seg.peer_array, mc, ctypes.c_longlong(off), ctypes.c_longlong(n_shard), self.rank,
                                                    self.world, L.ptr(dst), int(accumulate), ctypes.c_float(scale), L.ptr(norm_partials),
                                                    0 if norm_partials is None else norm_partials.numel(), ctypes.c_uint(seed & 0xFFFFFFFF),
                                                    self.sms, L.stream_ptr()), "p2p_reduce_scatter")

    # ---- GEMM with the reduce-scatter inside (csrc/gemm_tcgen05_2cta.cu)
    RS_COUNTER_BASE = MAX_CHANNELS * 8 * 4 + 2 * SMALL_SLOTS_FLOATS * 4       # counters live behind the small all-reduce slots

    def gemm_rs_supported(self, M: int, N: int) -> bool:
        return M % self.world == 0 and (M // self.world) % 32 == 0 and M >= 256 and N % 8 == 0

    def gemm_rs(self, landing: torch.Tensor, counter_id: int, dst: Optional[torch.Tensor], a: torch.Tensor, b: torch.Tensor, *, a_mn=False, b_mn=False,
                scale_a=None, scale_b=None, alpha: float = 1.0, prev: Optional[torch.Tensor] = None, shard_accumulate: bool = False,
                shard_scale: float = 1.0, norm_partials: Optional[torch.Tensor] = None, seed: int = 0) -> None:
        """dst (+)= shard_scale * (rows of this rank of the sum over ranks of (prev +) alpha * A @ B^T).

        One kernel: tcgen05 GEMM whose epilogue stores each output row into the owner rank's ``landing`` buffer
        ([world, M/world, N] bf16 in the heap, same allocation on every rank) and whose tail sums the slots.
        ``counter_id`` names the arrival counter of this landing buffer (one per buffer).  Callers make sure that every
        rank finished reading the previous content of its landing buffer (signal / wait) before the next call.

        ``dst=None``: the kernel only pushes (no waiting, no summing tail, nothing that changes from call to call, so it
        can sit in a CUDA graph); ``rs_finish`` on the collectives stream completes the reduce-scatter."""
        seg, off = self.heap.locate(landing)
        w = self.world
        M = landing.shape[0] * landing.shape[1]
        N = landing.shape[2]
        Kd = a.shape[0] if a_mn else a.shape[1]
        if not self.gemm_rs_supported(M, N) or landing.dtype != torch.bfloat16 or (dst is not None and dst.dtype != torch.bfloat16):
            raise ValueError("fused GEMM + reduce-scatter: unsupported shape or dtype")
        target = self._rs_next_target(counter_id, M, N) if dst is not None else 0
        ptrs = list(seg.hdl.buffer_ptrs)
        landing_arr = (ctypes.c_void_p * 8)(*([p + off for p in ptrs] + [0] * (8 - len(ptrs))))
        cptrs = list(self.ctrl.hdl.buffer_ptrs)
        coff = self.RS_COUNTER_BASE + 4 * counter_id
        counter_arr = (ctypes.c_void_p * 8)(*([p + coff for p in cptrs] + [0] * (8 - len(cptrs))))
        c_local = prev if prev is not None else landing
        rc = L.kernels().llmq_gemm_rs(
            L.ptr(a), L.ptr(b), L.ptr(c_local), M, N, Kd, L.dtype_code(a.dtype), L.dtype_code(b.dtype), int(a_mn), int(b_mn),
            ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), int(prev is not None), L.ptr(scale_a), L.ptr(scale_b),
            ctypes.c_float(alpha), L.ptr(self.status), self.sms, landing_arr, counter_arr, self.rank, w, ctypes.c_uint(target), L.ptr(dst),
            int(shard_accumulate), ctypes.c_float(shard_scale), L.ptr(norm_partials), 0 if norm_partials is None else norm_partials.numel(),
            ctypes.c_uint(seed & 0xFFFFFFFF), ctypes.c_double(self.wait_limit_s), L.stream_ptr())
        L.check(rc, "gemm_rs")

    def _rs_next_target(self, counter_id: int, M: int, N: int) -> int:
        """The value the local arrival counter reaches once every rank delivered all tiles of one more [M, N] product."""
        key = ("rs", counter_id)
        arrivals = int(L.kernels().llmq_gemm_rs_arrivals(M, N, self.world))
        target = (self.gen.get(key, 0) + arrivals) & 0xFFFFFFFF
        self.gen[key] = target
        return target

    def rs_finish(self, landing: torch.Tensor, counter_id: int, dst: torch.Tensor, *, accumulate: bool, scale: float,
                  norm_partials: Optional[torch.Tensor] = None, seed: int = 0) -> None:
        """Owner side of a push-only ``gemm_rs``: waits (bounded, on the device) for all sources' tiles of the landing buffer,
        then dst (+)= scale * sum of the local slots, with stochastic rounding and the squared-norm partials.  One call per
        ``gemm_rs(..., dst=None)`` on the same landing buffer, on the collectives stream."""
        M = landing.shape[0] * landing.shape[1]
        N = landing.shape[2]
        target = self._rs_next_target(counter_id, M, N)
        counter = ctypes.c_void_p(self.ctrl.base + self.RS_COUNTER_BASE + 4 * counter_id)
        L.check(L.kernels().llmq_p2p_rs_finish(L.ptr(landing), counter, ctypes.c_uint(target), ctypes.c_longlong(dst.numel()), self.rank,
                                               self.world, L.ptr(dst), int(accumulate), ctypes.c_float(scale), L.ptr(norm_partials),
                                               0 if norm_partials is None else norm_partials.numel(), ctypes.c_uint(seed & 0xFFFFFFFF),
                                               L.ptr(self.status), ctypes.c_double(self.wait_limit_s), self.sms, L.stream_ptr()), "p2p_rs_finish")

    def all_reduce_small(self, t: torch.Tensor, op: str = "sum") -> None:
        """In-place sum / max / avg of a few fp32 values across ranks, one kernel, no library call."""
        n = t.numel()
        if t.dtype != torch.float32 or not t.is_contiguous() or n > SMALL_SLOTS_FLOATS // self.world:
            raise ValueError("small all-reduce takes a contiguous fp32 tensor of limited size")
        gen = self.next_gen(self.small_channel)
        L.check(L.kernels().llmq_p2p_allreduce_small(self.ctrl.peer_array, ctypes.c_longlong(self.slots_offset),
                                                     ctypes.c_longlong(self._flag_offset(self.small_channel)), L.ptr(t), n, self.rank, self.world,
                                                     {"sum": 0, "max": 1, "avg": 2}[op], ctypes.c_uint(gen), L.ptr(self.status),
                                                     ctypes.c_double(self.wait_limit_s), L.stream_ptr()), "p2p_allreduce_small")
