"""ZeRO-style state managers: weights (master / work / quantised copies), gradients and AdamW moments.

Everything is sharded by contiguous row blocks of each tensor (dimension 0 must divide by the world size), the
layout used by the reference (src/utilities/tensor.cpp:113-120).  Capabilities mirror

* LLamaWeightsManager: gather / get / release with a versioned cache, unsharded (all layers resident) and
  sharded (two block buffers, ZeRO-3) flavours, quantise-before-gather, persistent quantised shards,
  master weights in pinned host memory (src/models/llama_weights.h:101-226, llama_weights.cpp);
* the gradient managers: full-replica gradients reduce-scattered on the last micro-step (ZeRO-1) or two block
  buffers reduce-scattered every micro-step and accumulated into per-layer shards with stochastic rounding
  (ZeRO-2) (src/training/gradients.cpp, src/models/llama_gradients.cpp);
* AdamWStateManager: 1/world shards of m and v, optionally in pinned host memory, with block scales for e4m3
  first moments (src/training/adamw_optimizer.cpp:161-221).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from types import SimpleNamespace
from typing import Dict, List, Optional

import torch

from ..config import TransformerConfig
from ..ops import kernels as K
from ..options import LLamaOptions
from ..utils import nvtx
from .comm import Communicator, _WorkList

F8_TYPES = (torch.float8_e4m3fn, torch.float8_e5m2)
MATRICES = ("qkv_w", "o_w", "up_w", "down_w")


@dataclass
class ParamSpec:
    name: str
    shape: tuple
    matrix: bool          # 2-D GEMM operand (quantised in fp8 mode, weight decay applies)
    init_std: float       # 0 -> zeros, <0 -> ones


def block_param_specs(cfg: TransformerConfig, opts: LLamaOptions) -> List[ParamSpec]:
    C, D, QC, L = cfg.hidden_size, cfg.intermediate_size, cfg.qkv_channels, cfg.num_hidden_layers
    proj_std = 0.0 if opts.init_projections_to_zero else 0.02 / (2 * L) ** 0.5
    specs = [ParamSpec("ln1_w", (C,), False, -1.0), ParamSpec("qkv_w", (QC, C), True, 0.02)]
    if cfg.use_qkv_bias:
        specs.append(ParamSpec("qkv_b", (QC,), False, 0.0))
    specs += [ParamSpec("o_w", (C, C), True, proj_std), ParamSpec("ln2_w", (C,), False, -1.0),
              ParamSpec("up_w", (2 * D, C), True, 0.02), ParamSpec("down_w", (C, D), True, proj_std)]
    return specs


def nonblock_param_specs(cfg: TransformerConfig) -> List[ParamSpec]:
    V, C = cfg.vocab_size, cfg.hidden_size
    specs = [ParamSpec("embed", (V, C), True, 0.02), ParamSpec("lnf_w", (C,), False, -1.0)]
    if not cfg.tie_word_embeddings:
        specs.append(ParamSpec("lm_head", (V, C), True, 0.02))
    return specs


_HOST_WRITE_COMBINED = False          # set by the managers from LLamaOptions.use_write_combined before they allocate


def _alloc(shape, dtype, device, pinned=False):
    if pinned:
        if _HOST_WRITE_COMBINED:
            from ..utils.memory import host_tensor
            return host_tensor(shape, dtype, write_combined=True)
        return torch.zeros(shape, dtype=dtype, pin_memory=torch.cuda.is_available())
    return torch.zeros(shape, dtype=dtype, device=device)


def _rows(shape, world):
    if shape[0] % world:
        raise ValueError(f"dimension 0 of a tensor of shape {shape} does not divide by the world size {world}")
    return (shape[0] // world,) + tuple(shape[1:])


# flag channels of the fused collectives (each channel = one word per source rank)
CH_WEIGHTS, CH_NONBLOCK, CH_GRADS, CH_GRADS_NB, CH_A2A = 0, 1024, 1100, 3000, 3500


class _FusedPending:
    """Handle of a fused gather / reduction: wait() orders the current stream after the side stream's work and
    after the arrival of every peer's data flag."""

    def __init__(self, fused, channel, gen, event, device):
        self.fused, self.channel, self.gen, self.event, self.device = fused, channel, gen, event, device

    def wait(self):
        torch.cuda.current_stream(self.device).wait_event(self.event)
        if self.channel is not None:
            self.fused.wait(self.channel, self.gen)


class _Buf:
    """One work buffer (a full transformer block) with its cache state."""

    def __init__(self):
        self.t: Dict[str, torch.Tensor] = {}
        self.layer = -1
        self.version = -1
        self.pending = None
        self.in_use = False


class WeightsManager:
    def __init__(self, cfg: TransformerConfig, opts: LLamaOptions, comm: Communicator, device: torch.device, fused=None):
        self.cfg, self.opts, self.comm, self.device = cfg, opts, comm, device
        global _HOST_WRITE_COMBINED
        _HOST_WRITE_COMBINED = bool(getattr(opts, "use_write_combined", False))      # offloaded tensors in write-combined pages
        self.fused = fused                    # FusedCollectives: gathers become in-kernel peer stores
        self.model_dtype = opts.model_type or cfg.dtype
        self.matmul_dtype = opts.matmul_dtype()
        self.master_dtype = opts.master()
        self.quantized = self.matmul_dtype in F8_TYPES
        self.sharded = bool(opts.shard_weights)
        self.block_specs = block_param_specs(cfg, opts)
        self.nonblock_specs = nonblock_param_specs(cfg)
        self.version = 0
        L, w = cfg.num_hidden_layers, comm.world
        host_master = opts.offload_master and device.type == "cuda"

        def work_dtype(s):
            return self.matmul_dtype if (s.matrix and s.name in MATRICES) else self.model_dtype

        # fused gathers need bf16 masters and bf16 / e4m3 work copies; masters in pinned host memory are staged to the
        # device first, kept e4m3 shards (--persistent-quants) are pushed as they are
        if self.fused is not None and not (self.master_dtype == torch.bfloat16 and self.model_dtype == torch.bfloat16
                                           and self.matmul_dtype in (torch.bfloat16, torch.float8_e4m3fn)):
            self.fused = None
        walloc = (lambda shape, dt: self.fused.heap.empty(shape, dt)) if self.fused is not None else (lambda shape, dt: _alloc(shape, dt, device))
        # ---- work buffers
        n_bufs = 2 if self.sharded else L
        self.bufs = [_Buf() for _ in range(n_bufs)]
        for b in self.bufs:
            for s in self.block_specs:
                b.t[s.name] = walloc(s.shape, work_dtype(s))
        self.nb_work: Dict[str, torch.Tensor] = {}
        for s in self.nonblock_specs:
            if self.sharded and s.name == "lm_head":
                continue                      # embedding and head share one gather buffer under ZeRO-3
            self.nb_work[s.name] = walloc(s.shape, self.model_dtype)
        self.nb_state = {"embed": [-1, None], "lnf_w": [-1, None], "emb_slot_holds": None}

        # ---- master shards
        self.master_blocks: List[Dict[str, torch.Tensor]] = []
        for l in range(L):
            d = {}
            for s in self.block_specs:
                alias = (not self.sharded) and work_dtype(s) == self.master_dtype and not host_master
                if alias:
                    d[s.name] = comm.local_shard(self.bufs[l].t[s.name])
                else:
                    d[s.name] = _alloc(_rows(s.shape, w), self.master_dtype, device, pinned=host_master)
            self.master_blocks.append(d)
        self.master_nb: Dict[str, torch.Tensor] = {}
        for s in self.nonblock_specs:
            alias = (not self.sharded) and self.model_dtype == self.master_dtype and not host_master
            if alias:
                self.master_nb[s.name] = comm.local_shard(self.nb_work[s.name])
            else:
                self.master_nb[s.name] = _alloc(_rows(s.shape, w), self.master_dtype, device, pinned=host_master)

        # ---- persistent quantised shards (ZeRO-3 option)
        self.quant_shards: Optional[List[Dict[str, torch.Tensor]]] = None
        self.quant_version = [-1] * L
        if self.sharded and opts.persistent_quants and self.quantized:
            pin = opts.offload_quants and device.type == "cuda"
            self.quant_shards = [{n: _alloc(_rows(s.shape, w), self.matmul_dtype, device, pinned=pin)
                                  for s in self.block_specs if (n := s.name) in MATRICES} for _ in range(L)]

        # ---- abs-max / dequant-scale table: [layer, matrix, {absmax, scale}]
        self.w_stats = torch.zeros(L, len(MATRICES), 2, dtype=torch.float32, device=device)
        self._staging: Dict[str, torch.Tensor] = {}

    # ------------------------------------------------------------------ helpers
    def _stat(self, l, name):
        return self.w_stats[l, MATRICES.index(name)]

    def _to_device(self, t: torch.Tensor, key: str) -> torch.Tensor:
        """Pinned-host tensors are staged through a reusable device buffer (H2D on the current stream)."""
        if t.device.type == self.device.type:
            return t
        st = self._staging.get(key)
        if st is None or st.shape != t.shape or st.dtype != t.dtype:
            st = torch.empty(t.shape, dtype=t.dtype, device=self.device)
            self._staging[key] = st
        st.copy_(t, non_blocking=True)
        return st

    def invalidate(self) -> None:
        """Called after the optimizer changed the master weights: cached work copies are stale."""
        self.version += 1

    # ------------------------------------------------------------------ blocks
    def _buf_for(self, l) -> _Buf:
        return self.bufs[l % 2] if self.sharded else self.bufs[l]

    def gather_block(self, l: int) -> None:
        buf = self._buf_for(l)
        if buf.layer == l and buf.version == self.version:
            return
        if buf.in_use:
            raise RuntimeError(f"weight buffer for layer {l} is still in use by layer {buf.layer}")
        with nvtx.range(f"gather_block {l}", self.device):
            self._gather_block(l, buf)

    def _gather_block(self, l: int, buf) -> None:
        if self.fused is not None and self.comm.world > 1:
            self._gather_block_fused(l, buf)
            return
        works = []
        for s in self.block_specs:
            full = buf.t[s.name]
            local = self.comm.local_shard(full)
            master = self.master_blocks[l][s.name]
            if s.name in MATRICES and self.quantized:
                st = self._stat(l, s.name)
                if self.quant_shards is not None:
                    q = self.quant_shards[l][s.name]
                    if self.quant_version[l] != self.version:
                        K.quantize(local, st[1:2], self._to_device(master, "m_" + s.name), st[0:1])
                        q.copy_(local, non_blocking=True)      # kept (device or pinned host) for later gathers
                    else:
                        local.copy_(q, non_blocking=True)
                else:
                    K.quantize(local, st[1:2], self._to_device(master, "m_" + s.name), st[0:1])
            elif master.data_ptr() != local.data_ptr():
                local.copy_(self._to_device(master, "m_" + s.name))
            if self.comm.world > 1:
                works.append(self.comm.all_gather(full, local))
        if self.quant_shards is not None:
            self.quant_version[l] = self.version
        buf.pending = _WorkList(works)
        buf.ready = None
        buf.layer, buf.version = l, self.version

    def _gather_block_fused(self, l: int, buf: _Buf) -> None:
        """Quantise-and-push: every rank stores its (quantised) shard straight into all ranks' buffers over NVLink.
        Side stream: barrier (all ranks are past the previous user of this buffer) -> pushes -> data flag."""
        f = self.fused
        idx = self.bufs.index(buf)
        ch_free, ch_vec, ch_mat = CH_WEIGHTS + 3 * idx, CH_WEIGHTS + 3 * idx + 1, CH_WEIGHTS + 3 * idx + 2
        main = torch.cuda.current_stream(self.device)
        f.stream.wait_stream(main)
        with torch.cuda.stream(f.stream):
            f.wait(ch_free, f.signal(ch_free))
            # the small vectors first: their flag is awaited by a tiny kernel before the layer starts; the matrices'
            # flags are polled by the consuming GEMMs themselves, tile by tile
            memcpy = bool(getattr(self.opts, "memcpy_all_gather", False))     # copy engines instead of SM stores for the pushes
            for s in self.block_specs:
                if s.name not in MATRICES:
                    src = self._to_device(self.master_blocks[l][s.name], "m_" + s.name)
                    if memcpy:
                        self.comm.local_shard(buf.t[s.name]).copy_(src)
                        f.copy_allgather(buf.t[s.name])
                    else:
                        f.quant_allgather(buf.t[s.name], src)
            gen_vec = f.signal(ch_vec)
            for s in self.block_specs:
                if s.name in MATRICES:
                    full = buf.t[s.name]
                    master = self.master_blocks[l][s.name]
                    if self.quantized:
                        st = self._stat(l, s.name)
                        q = self.quant_shards[l][s.name] if self.quant_shards is not None else None
                        if memcpy:
                            # quantise (or fetch the kept shard) into the own slot, then copy-engine transfers to the peers
                            local = self.comm.local_shard(full)
                            if q is not None and self.quant_version[l] == self.version:
                                local.copy_(q, non_blocking=True)
                            else:
                                K.quantize(local, st[1:2], self._to_device(master, "m_" + s.name), st[0:1])
                                if q is not None:
                                    q.copy_(local, non_blocking=True)
                            f.copy_allgather(full)
                        elif q is not None and self.quant_version[l] == self.version:
                            # kept e4m3 shard: the master is not read again (a shard in pinned host memory is staged first)
                            f.push_allgather(full, self._to_device(q, "q_" + s.name))
                        else:
                            f.quant_allgather(full, self._to_device(master, "m_" + s.name), st[0:1], st[1:2])
                            if q is not None:
                                q.copy_(self.comm.local_shard(full), non_blocking=True)      # own slot, as just pushed
                    elif memcpy:
                        self.comm.local_shard(full).copy_(self._to_device(master, "m_" + s.name))
                        f.copy_allgather(full)
                    else:
                        f.quant_allgather(full, self._to_device(master, "m_" + s.name))
            if self.quant_shards is not None:
                self.quant_version[l] = self.version
            gen_mat = f.signal(ch_mat)
            ev = torch.cuda.Event()
            ev.record(f.stream)
        if os.environ.get("LLMQ_GEMM_POLL", "0") != "1":
            # Default: one wait kernel for the whole block in front of the layer.  With the prefetch depth of one layer
            # the data has long arrived, and polling the flags inside every GEMM measured 30 ms / step slower on
            # Qwen2.5-7B (571 vs 540 ms, 2 GPUs); LLMQ_GEMM_POLL=1 switches the in-GEMM polling on.
            buf.pending = _FusedPending(f, ch_mat, gen_mat, ev, self.device)
            buf.ready = None
        else:
            buf.pending = _FusedPending(f, ch_vec, gen_vec, ev, self.device)
            buf.ready = {n: (f.ctrl.base + f._flag_offset(ch_mat), gen_mat, buf.t[n].shape[0] // self.comm.world, f.wait_limit_s)
                         for n in MATRICES}
        buf.layer, buf.version = l, self.version

    def get_block(self, l: int) -> SimpleNamespace:
        buf = self._buf_for(l)
        if buf.layer != l or buf.version != self.version:
            raise RuntimeError(f"gathered data is not for the requested layer {l} (have {buf.layer})")
        if buf.pending is not None:
            buf.pending.wait()
            buf.pending = None
        buf.in_use = True
        ns = SimpleNamespace(**buf.t)
        ns.ready = getattr(buf, "ready", None) or {n: None for n in MATRICES}
        ns.scales = {n: self._stat(l, n)[1:2] for n in MATRICES} if self.quantized else {n: None for n in MATRICES}
        if not hasattr(ns, "qkv_b"):
            ns.qkv_b = None
        return ns

    def release_block(self, l: int) -> None:
        self._buf_for(l).in_use = False

    # ------------------------------------------------------------------ non-block tensors
    def _gather_nb(self, name: str, slot: str) -> torch.Tensor:
        full = self.nb_work[slot]
        st = self.nb_state.setdefault(slot, [-1, None])
        holds = self.nb_state.get("holds_" + slot, slot)
        if st[0] == self.version and holds == name:
            return full
        local = self.comm.local_shard(full)
        master = self.master_nb[name]
        if self.fused is not None and self.comm.world > 1:
            f = self.fused
            ch = CH_NONBLOCK + 2 * list(self.nb_work).index(slot)
            f.wait(ch, f.signal(ch))                     # every rank is done with the slot's previous content
            if getattr(self.opts, "memcpy_all_gather", False):
                local.copy_(self._to_device(master, "nb_" + name))
                f.copy_allgather(full)
            else:
                f.quant_allgather(full, self._to_device(master, "nb_" + name))
            f.wait(ch + 1, f.signal(ch + 1))
        else:
            if master.data_ptr() != local.data_ptr():
                local.copy_(self._to_device(master, "nb_" + name))
            if self.comm.world > 1:
                st[1] = self.comm.all_gather(full, local)
        st[0] = self.version
        self.nb_state["holds_" + slot] = name
        return full

    def _wait_nb(self, slot):
        st = self.nb_state.get(slot)
        if st and st[1] is not None:
            st[1].wait()
            st[1] = None

    def get_embeddings(self) -> torch.Tensor:
        t = self._gather_nb("embed", "embed")
        self._wait_nb("embed")
        return t

    def get_head(self) -> torch.Tensor:
        if self.cfg.tie_word_embeddings:
            return self.get_embeddings()
        slot = "embed" if self.sharded else "lm_head"
        t = self._gather_nb("lm_head", slot)
        self._wait_nb(slot)
        return t

    def get_lnf(self) -> torch.Tensor:
        t = self._gather_nb("lnf_w", "lnf_w")
        self._wait_nb("lnf_w")
        return t

    # ------------------------------------------------------------------ abs-max bookkeeping
    def zero_absmax(self) -> None:
        self.w_stats[:, :, 0].zero_()

    def sync_absmax(self, recompute: bool) -> None:
        """All ranks must quantise a matrix with the same scale: max-reduce the per-shard abs-max values."""
        if not self.quantized:
            return
        if recompute:
            self.zero_absmax()
            for l in range(self.cfg.num_hidden_layers):
                for n in MATRICES:
                    K.abs_max(self._stat(l, n)[0:1], self._to_device(self.master_blocks[l][n], "m_" + n))
        if self.comm.world > 1:
            am = self.w_stats[:, :, 0].contiguous()
            if self.fused is not None and am.numel() * self.comm.world <= 4096:
                self.fused.all_reduce_small(am.view(-1), "max")
            else:
                self.comm.all_reduce(am, "max").wait()
            self.w_stats[:, :, 0].copy_(am)

    # ------------------------------------------------------------------ iteration (checkpoint / optimizer)
    def master_items(self):
        """Yields (checkpoint name, master shard, spec, layer or None) for every parameter."""
        for l, d in enumerate(self.master_blocks):
            for s in self.block_specs:
                yield f"layers.{l}.{s.name}", d[s.name], s, l
        for s in self.nonblock_specs:
            yield s.name, self.master_nb[s.name], s, None


class GradientManager:
    """Full or sharded gradient storage plus the reduction protocol
    start_micro_step -> get_block_full -> notify_block -> end_micro_step -> get_block_shard."""

    def __init__(self, cfg, opts, comm: Communicator, device, weights: WeightsManager, seed: int = 42):
        self.cfg, self.opts, self.comm, self.device = cfg, opts, comm, device
        self.dtype = weights.model_dtype
        self.block_specs, self.nonblock_specs = weights.block_specs, weights.nonblock_specs
        self.sharded = bool(opts.shard_gradients)
        self.seed, self.step = seed, 0
        L, w = cfg.num_hidden_layers, comm.world
        host = opts.offload_grads and device.type == "cuda" and self.sharded
        self.micro_step, self.last = 0, False
        # in-kernel reduce-scatter: bf16 gradients in the symmetric heap, shards on the device
        self.fused = weights.fused if (weights.fused is not None and self.dtype == torch.bfloat16 and not host and w > 1) else None
        self.norm_fused = self.fused is not None
        # squared-norm partials: first half written by the side-stream reductions, second half by GEMMs with the
        # reduce-scatter inside (main stream), so the two streams never touch the same word
        self.norm_partials = torch.zeros(2 * K.NORM_PARTIALS, dtype=torch.float32, device=device) if self.fused is not None else None
        # Weight-gradient GEMMs start their reduce-scatter in the epilogue: every output tile is pushed into the owner
        # rank's landing buffer over NVLink while the tensor core works on the next tile; the owner-side sum (1/world,
        # stochastic-rounding accumulation, norm partials) is one small kernel per matrix on the collectives stream that waits
        # for its arrival counter (`_rs_finishers`).  Default; LLMQ_GEMM_RS=0 selects the plain GEMM followed by the pull
        # reduce-scatter kernel.  Qwen2.5-7B, 2 GPUs, same box, alternating runs: 473.9 / 474.1 ms against 477.6 / 478.3 ms.
        # (An earlier form that summed inside the GEMM kernel's tail held all SMs while it waited for the peers and lost.)
        self.gemm_rs = self.fused is not None and os.environ.get("LLMQ_GEMM_RS", "1") == "1"
        # --all-to-all-reduce with --memcpy-send-recv (LLamaGradientsBlockSharded_AllToAll with memcpy transfers in the
        # reference, llama_gradients.cpp:81-134): plain GEMMs, then copy-engine transfers of slot s to rank s's landing buffer
        # and a local sum.  Without --memcpy-send-recv the all-to-all is the GEMM epilogue's push above (SM stores).
        self.a2a_copy = bool(self.fused is not None and self.sharded and opts.use_all_to_all_reduce and getattr(opts, "memcpy_send_recv", False))
        if self.a2a_copy:
            self.gemm_rs = False
        self._fdone: Dict[int, tuple] = {}           # channel -> (generation, event) of the last reduction reading a buffer
        self._fevents: List = []
        _heap = self.fused.heap if self.fused is not None else None
        _galloc = (lambda shape: _heap.empty(shape, self.dtype)) if _heap is not None else (lambda shape: _alloc(shape, self.dtype, device))
        if self.sharded:
            self.bufs = [{s.name: _galloc(s.shape) for s in self.block_specs} for _ in range(2)]
            self.buf_state = [{"layer": -1, "pending": None, "needs_acc": False} for _ in range(2)]
            self.shards = [{s.name: _alloc(_rows(s.shape, w), self.dtype, device, pinned=host) for s in self.block_specs}
                           for _ in range(L)]
        else:
            self.full = [{s.name: _galloc(s.shape) for s in self.block_specs} for _ in range(L)]
            self.pending: List = [None] * L
        self.a2a_landing = ([{s.name: _galloc(s.shape) for s in self.block_specs if s.matrix and s.shape[0] % w == 0} for _ in range(2)]
                            if self.a2a_copy else None)
        self.nb_full = {s.name: _galloc(s.shape) for s in self.nonblock_specs}
        self.nb_pending: Dict[str, object] = {}
        self._stage: Dict[str, torch.Tensor] = {}

    # -- micro-step protocol
    def start_micro_step(self, micro_step: int, total: int) -> None:
        self.micro_step, self.last = micro_step, micro_step == total - 1
        if micro_step == 0 and self.fused is not None:
            for k in range(len(self.nonblock_specs)):          # peers may still read last step's non-block gradients
                self._wait_readers(CH_GRADS_NB + 2 * k)
        if micro_step == 0:
            for s in self.nonblock_specs:
                if not s.matrix:
                    self.nb_full[s.name].zero_()

    def get_block_full(self, l: int):
        """Returns (tensors, accumulate): where layer l's backward writes, and whether it adds to the content."""
        if self.fused is not None:
            self._wait_readers(CH_GRADS + 2 * (l % 2 if self.sharded else l))
        if not self.sharded:
            g = self.full[l]
            acc = self.micro_step > 0
        else:
            i = l % 2
            if self.fused is None:
                self._flush(i)
            g = self.bufs[i]
            self.buf_state[i]["layer"] = l
            acc = False
        if not acc:
            for s in self.block_specs:
                if not s.matrix:
                    g[s.name].zero_()          # vectors are always accumulated into; matrices are overwritten
        return g, acc

    # -- fused (in-kernel) reduction -------------------------------------------------------------
    def _wait_readers(self, ch_ready: int) -> None:
        """Before a gradient buffer is overwritten: our own reduction and every peer's reads of it are finished."""
        d = self._fdone.pop(ch_ready, None)
        if d is not None:
            gen, ev = d
            torch.cuda.current_stream(self.device).wait_event(ev)
            self.fused.wait(ch_ready + 1, gen)

    def _reduce_fused(self, ch_ready: int, pairs, accumulate: bool, seed: int, finishers=(), a2a=(), ch_a2a: int = 0) -> None:
        """pairs: [(full tensor in the heap, destination shard)].  Main stream: flag "my gradients are complete".
        Side stream: the owner-side halves of the in-GEMM reduce-scatters (``finishers``: each waits for its own arrival
        counter), then wait for every rank's flag, pull-and-reduce this rank's rows, flag "done reading"."""
        f = self.fused
        main = torch.cuda.current_stream(self.device)
        gen = f.signal(ch_ready)
        f.stream.wait_stream(main)
        with torch.cuda.stream(f.stream):
            for fin in finishers:
                fin()
            if a2a:
                # copy-engine all-to-all: every peer finished with its landing buffers before this block's backward began
                # (get_block_full waited for all ranks' "done reading" flags), so the transfers can start right away
                for full, landing, dst, sd in a2a:
                    f.copy_all_to_all(full, landing)
                f.wait(ch_a2a, f.signal(ch_a2a))             # every rank's slots have landed everywhere
                w = self.comm.world
                for full, landing, dst, sd in a2a:
                    f.sum_slots(landing.view(w, -1), dst, accumulate=accumulate, scale=1.0 / w,
                                norm_partials=self.norm_partials[:K.NORM_PARTIALS] if self.last else None, seed=sd)
            f.wait(ch_ready, gen)
            for k, (full, dst) in enumerate(pairs):
                f.reduce_scatter(full, dst, accumulate=accumulate, scale=1.0 / self.comm.world,
                                 norm_partials=self.norm_partials[:K.NORM_PARTIALS] if self.last else None, seed=seed + 17 * k)
            done = f.signal(ch_ready + 1)
            ev = torch.cuda.Event()
            ev.record(f.stream)
        self._fdone[ch_ready] = (done, ev)
        self._fevents.append(ev)

    def _block_seed(self, l: int) -> int:
        return (self.seed * 7919 + self.step * 104729 + l * 131 + self._acc_count[l] * 7) & 0x7FFFFFFF

    def _rs_plan(self, l: int, name: str):
        """(landing buffer, counter id, destination shard, accumulate) when the weight gradient ``name`` of layer ``l`` is
        reduce-scattered from inside its GEMM in the current micro-step, else None.  Depends only on the step state, not
        on whether the block body was executed by Python or replayed from a CUDA graph."""
        if not self.gemm_rs or not (self.sharded or (self.last and self.micro_step == 0)):
            return None
        k = next(i for i, s in enumerate(self.block_specs) if s.name == name)
        spec = self.block_specs[k]
        if not spec.matrix or not self.fused.gemm_rs_supported(spec.shape[0], spec.shape[1]):
            return None
        w = self.comm.world
        M, N = spec.shape
        if self.sharded:
            i = l % 2
            return self.bufs[i][name].view(w, M // w, N), i * 16 + k, self.shards[l][name], self._acc_count[l] > 0, k
        full = self.full[l][name]                           # the own slot of the landing buffer is the shard itself
        return full.view(w, M // w, N), 64 + l * 16 + k, self.comm.local_shard(full), False, k

    def fused_dw(self, l: int, name: str):
        """A callable ``run(a, b, scale_a, scale_b)`` that computes this rank's weight gradient ``a^T-stored @ b`` with a
        GEMM whose epilogue pushes every output row into the owner rank's landing buffer over NVLink (the reduce-scatter
        starts tile by tile inside the GEMM; ``notify_block`` finishes it on the collectives stream), or ``None`` when the
        plain GEMM has to be used: no peer-memory path, the reduction does not follow this micro-step, or the shape does
        not split into row shards of a multiple of 32 rows."""
        plan = self._rs_plan(l, name)
        if plan is None:
            return None
        landing, counter = plan[0], plan[1]

        def run(a, b, scale_a=None, scale_b=None, a_mn=True, b_mn=True):
            self.fused.gemm_rs(landing, counter, None, a, b, a_mn=a_mn, b_mn=b_mn, scale_a=scale_a, scale_b=scale_b)
        return run

    def _rs_finishers(self, l: int):
        """The owner-side halves of this block's in-GEMM reduce-scatters: callables for the collectives stream."""
        out, names = [], set()
        for s in self.block_specs:
            plan = self._rs_plan(l, s.name) if s.matrix else None
            if plan is None:
                continue
            landing, counter, dst, acc, k = plan
            seed = self._block_seed(l) + 17 * k
            parts = self.norm_partials[:K.NORM_PARTIALS] if self.last else None
            names.add(s.name)
            out.append(lambda landing=landing, counter=counter, dst=dst, acc=acc, seed=seed, parts=parts: self.fused.rs_finish(
                landing, counter, dst, accumulate=acc, scale=1.0 / self.comm.world, norm_partials=parts, seed=seed))
        return out, names

    def notify_block(self, l: int) -> None:
        if self.fused is not None:
            seed = self._block_seed(l)
            finishers, done = self._rs_finishers(l)          # matrices whose reduce-scatter started inside their GEMM
            if not self.sharded:
                if self.last:
                    self._reduce_fused(CH_GRADS + 2 * l, [(t, self.comm.local_shard(t)) for n, t in self.full[l].items() if n not in done],
                                       False, seed, finishers)
            else:
                i = l % 2
                a2a = []
                if self.a2a_copy:
                    for k, s in enumerate(self.block_specs):
                        if s.name in self.a2a_landing[i]:
                            a2a.append((self.bufs[i][s.name], self.a2a_landing[i][s.name], self.shards[l][s.name], seed + 17 * k))
                            done.add(s.name)
                pairs = [(self.bufs[i][s.name], self.shards[l][s.name]) for s in self.block_specs if s.name not in done]
                self._reduce_fused(CH_GRADS + 2 * i, pairs, self._acc_count[l] > 0, seed, finishers, a2a, CH_A2A + i)
                self._acc_count[l] += 1
            return
        if not self.sharded:
            if self.last and self.comm.world > 1:
                self.pending[l] = _WorkList([self.comm.reduce_scatter_avg(t) for t in self.full[l].values()])
            return
        i = l % 2
        st = self.buf_state[i]
        if self.comm.world > 1:
            st["pending"] = _WorkList([self.comm.reduce_scatter_avg(t) for t in self.bufs[i].values()])
        st["needs_acc"] = True

    def _flush(self, i: int) -> None:
        """Accumulates the reduced local slice of buffer i into the persistent shard of its layer."""
        st = self.buf_state[i]
        if not st["needs_acc"]:
            return
        if st["pending"] is not None:
            st["pending"].wait()
            st["pending"] = None
        l = st["layer"]
        for k, s in enumerate(self.block_specs):
            src = self.comm.local_shard(self.bufs[i][s.name])
            dst = self.shards[l][s.name]
            on_dev = dst.device.type == self.device.type
            if self.micro_step_of_layer_first(l):
                dst.copy_(src, non_blocking=True)
            else:
                d = dst if on_dev else self._staged(dst, s.name)
                seed = (self.seed * 7919 + self.step * 104729 + l * 131 + k * 17 + self._acc_count[l]) & 0x7FFFFFFF
                if d.numel() % 8 == 0 and d.dtype in (torch.bfloat16, torch.float32):
                    K.vector_add_sr(d, d, src, 1.0, seed)
                else:
                    d.add_(src)
                if not on_dev:
                    dst.copy_(d, non_blocking=True)
        self._acc_count[l] += 1
        st["needs_acc"] = False

    def _staged(self, host_t, key):
        st = self._stage.get(key)
        if st is None or st.shape != host_t.shape:
            st = torch.empty(host_t.shape, dtype=host_t.dtype, device=self.device)
            self._stage[key] = st
        st.copy_(host_t, non_blocking=True)
        return st

    def micro_step_of_layer_first(self, l: int) -> bool:
        return self._acc_count[l] == 0

    def begin_step(self) -> None:
        self._acc_count = [0] * self.cfg.num_hidden_layers
        if self.norm_partials is not None:
            self.norm_partials.zero_()

    def notify_non_block(self, name: str) -> None:
        if self.fused is not None:
            if self.last:
                k = [s.name for s in self.nonblock_specs].index(name)
                t = self.nb_full[name]
                self._reduce_fused(CH_GRADS_NB + 2 * k, [(t, self.comm.local_shard(t))], False, 0)
            return
        if self.last and self.comm.world > 1:
            self.nb_pending[name] = self.comm.reduce_scatter_avg(self.nb_full[name])

    def end_micro_step(self) -> None:
        if self.sharded and self.fused is None:
            self._flush(0)
            self._flush(1)

    def end_step(self) -> None:
        self.step += 1

    # -- optimizer side
    def wait_all(self) -> None:
        if self.fused is not None:
            main = torch.cuda.current_stream(self.device)
            for ev in self._fevents:
                main.wait_event(ev)
            self._fevents = []
            return
        if not self.sharded:
            for l, p in enumerate(self.pending):
                if p is not None:
                    p.wait()
                    self.pending[l] = None
        for n in list(self.nb_pending):
            self.nb_pending.pop(n).wait()

    def get_block_shard(self, l: int) -> Dict[str, torch.Tensor]:
        if self.sharded:
            return self.shards[l]
        return {n: self.comm.local_shard(t) for n, t in self.full[l].items()}

    def get_nb_shard(self, name: str) -> torch.Tensor:
        return self.comm.local_shard(self.nb_full[name])


class OptimizerStateManager:
    """AdamW first / second moments as 1/world row shards of every parameter."""

    def __init__(self, cfg, opts: LLamaOptions, comm, device, weights: WeightsManager):
        self.opts, self.device = opts, device
        self.m_dtype, self.v_dtype = opts.momentum_type, opts.variance_type
        self.m: Dict[str, torch.Tensor] = {}
        self.v: Dict[str, torch.Tensor] = {}
        self.m_scales: Dict[str, torch.Tensor] = {}
        pin_m = opts.offload_opt_m and device.type == "cuda"
        pin_v = opts.offload_opt_v and device.type == "cuda"
        for name, master, spec, l in weights.master_items():
            self.m[name] = _alloc(master.shape, self.m_dtype, device, pinned=pin_m)
            self.v[name] = _alloc(master.shape, self.v_dtype, device, pinned=pin_v)
            if self.m_dtype in F8_TYPES:
                n = master.numel()
                if n % 128:
                    raise ValueError(f"e4m3 momentum needs shard sizes divisible by 128 (tensor {name} has {n})")
                # scale blocks are 128 consecutive elements of the flat shard, independent of the world size
                self.m_scales[name] = torch.ones(n // 128, dtype=torch.float32, device=device)

    def items(self):
        for name in self.m:
            yield name, self.m[name], self.v[name], self.m_scales.get(name)
