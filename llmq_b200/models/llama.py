"""Llama / Qwen2 decoder with hand-scheduled forward, backward and optimizer step (no autograd).

The step structure follows the reference model (src/models/llama_model.cpp:73-894): ``forward`` runs the
blocks and the final norm, ``backward`` runs the (chunked) LM head with the fused classifier, then the blocks
in reverse with optional recomputation, and ``update`` clips by the global gradient norm and applies AdamW to
the local shards.  What differs is how the work is mapped to the hardware: every GEMM is the tcgen05 kernel
reading operands in their natural layout (MN-major descriptors take the place of the transpose kernels of the
fp8 backward recipe, llama_model.cpp:309-339), attention is the tcgen05 flash kernel on the packed QKV
tensor, and quantisation uses per-tensor just-in-time scaling with abs-max values produced by the preceding
kernel's epilogue.

Weight layout (llama_weights.cpp:915-938): q/k/v are fused row-wise into ``qkv_w`` [QC, C] (+ ``qkv_b``), up and
gate into ``up_w`` [2D, C] (up first), embeddings may be tied to the LM head.
"""
from __future__ import annotations

import os

from types import SimpleNamespace
from typing import Dict, List, Optional

import torch

from ..config import TransformerConfig
from ..ops import kernels as K
from ..options import LLamaOptions
from ..parallel.comm import Communicator, LocalComm
from ..parallel.offload import ResidualStore, Stager
from ..utils import nvtx
from ..parallel.zero import F8_TYPES, MATRICES, GradientManager, OptimizerStateManager, WeightsManager

# abs-max slots per layer: index -> (absmax, scale)
S_LN1, S_ATT, S_LN2, S_SWIGLU, S_DRESFFN, S_DMLPUP, S_DRESATT, S_DQKV = range(8)
N_SLOTS = 16


class _BlockGraphs:
    """CUDA graphs of the per-layer forward and recompute + backward bodies (``--use-cuda-graphs``).

    Every layer works on its own fixed buffers, so each (phase, layer, accumulate) body is captured once - on its
    second execution, after an eager warm-up run - and replayed afterwards; one replay stands for the ~20-45 kernel
    launches of a block.  Role of the per-block capture / update in the reference (llama_model.cpp:120-176,403-459).
    """

    def __init__(self, device: torch.device):
        self.device = device
        self.stream = torch.cuda.Stream(device)
        self.graphs: Dict[tuple, tuple] = {}
        self.warm: set = set()

    def run(self, key: tuple, fn) -> None:
        from ..ops import lib as _L
        entry = self.graphs.get(key)
        if entry is None:
            if key not in self.warm:                       # first time: plain launches (lazy one-time set-up happens here)
                self.warm.add(key)
                fn()
                return
            graph = torch.cuda.CUDAGraph()
            before = _L.launch_count
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.graph(graph, stream=self.stream):
                fn()
            entry = (graph, _L.launch_count - before)
            _L.launch_count = before                       # capturing launched nothing
            self.graphs[key] = entry
        entry[0].replay()
        _L.launch_count += entry[1]


class LlamaModel:
    def __init__(self, cfg: TransformerConfig, opts: LLamaOptions, comm: Optional[Communicator] = None,
                 device: Optional[torch.device] = None, batch_size: int = 1, seq_len: int = 128):
        cfg.validate()
        self.cfg, self.opts = cfg, opts
        self.comm = comm or LocalComm()
        self.device = torch.device(device) if device is not None else torch.device("cpu")
        if opts.model_type is None:
            opts.model_type = cfg.dtype
        self.dtype = opts.model_type
        self.B, self.T = batch_size, seq_len
        # GEMM operands in their own dtype: fp8 (per-tensor scaled), or bf16 under an fp32 model (mixed precision: scale 1)
        self.quant = opts.matmul_dtype() in F8_TYPES or (opts.matmul_dtype() == torch.bfloat16 and self.dtype == torch.float32)
        self.qdtype = opts.matmul_dtype()
        self.gdtype = opts.grad_dtype() if self.quant else self.dtype
        # block-scaled e4m3: bf16 plumbing, every block GEMM quantises its operands per 32 elements of its contraction axis
        self.mx = bool(opts.block_scaled)
        if self.mx:
            if self.quant or self.dtype != torch.bfloat16:
                raise ValueError("block_scaled needs a bf16 model without a per-tensor fp8 matmul_type")
            dims = {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size, "qkv_channels": cfg.qkv_channels,
                    "batch * seq_len": batch_size * seq_len}
            bad = [f"{k}={v}" for k, v in dims.items() if v % 128]
            if bad:
                raise ValueError("block_scaled needs contraction lengths that are multiples of 128: " + ", ".join(bad))
            if os.environ.get("LLMQ_GEMM_POLL", "0") == "1":
                raise ValueError("block_scaled quantises whole weight matrices and cannot poll for arriving weight rows (LLMQ_GEMM_POLL)")
        if seq_len > cfg.max_position_embeddings:
            raise ValueError("sequence length exceeds max_position_embeddings")
        self.fused = self._make_fused()
        self._marks: List = []
        # second stream: weight-gradient GEMMs of the blocks (overlap_dw) and the LM-head gradient GEMMs of a chunk beside the
        # next chunk's logits + classifier (overlap_lmhead)
        self._side_stream = (torch.cuda.Stream(self.device, priority=-1)
                             if ((opts.overlap_dw or opts.overlap_lmhead) and self.device.type == "cuda") else None)
        self._dw_stream = self._side_stream if opts.overlap_dw else None
        self._mx_dw_event = None                  # block-scaled path: last weight-gradient GEMM that reads the shared operand buffers
        self._dw_events: List = []
        # SwiGLU inside the epilogues of the up-projection GEMM and of the down-projection's dX GEMM
        self._fuse_swiglu = (opts.fuse_swiglu and not self.mx and self.device.type == "cuda" and self.dtype == torch.bfloat16
                             and batch_size * seq_len >= 256 and cfg.intermediate_size % 128 == 0)
        # per-block CUDA graphs: only where a block body contains nothing but kernels on fixed buffers
        self.graphs = None
        if (opts.use_cuda_graphs and self.device.type == "cuda" and not opts.offload_residual
                and os.environ.get("LLMQ_GEMM_POLL", "0") != "1"):
            self.graphs = _BlockGraphs(self.device)
        # sharded weights on several GPUs: each block body runs as two parts with the next block's weight gather started between them
        self._split_blocks = bool(self.comm.world > 1 and opts.shard_weights and opts.gather_behind_first_gemm)
        self.weights = WeightsManager(cfg, opts, self.comm, self.device, self.fused)
        self.grads = GradientManager(cfg, opts, self.comm, self.device, self.weights)
        self.opt_state = OptimizerStateManager(cfg, opts, self.comm, self.device, self.weights)
        self._alloc_run_state()
        self._stager = Stager(self.device, zero_copy=bool(opts.use_zero_copy))
        self.adam_seed = 42
        self.rng_state = 42                       # advanced every optimizer step; saved in checkpoints

    def _make_fused(self):
        """In-kernel NVLink collectives when asked for ("fused") or possible ("auto"): several ranks, one per process,
        CUDA devices with symmetric-memory support.  "nccl" keeps the library collectives."""
        mode = self.opts.collectives
        if self.dtype == torch.float32 and self.comm.world > 1 and mode != "nccl":
            # the peer-memory kernels move bf16 / fp8 tensors; fp32 models use the library collectives
            if mode == "fused":
                raise RuntimeError("fused collectives are not available for fp32 models; use collectives='nccl'")
            return None
        if mode == "nccl" or self.comm.world == 1 or self.device.type != "cuda" or not hasattr(self.comm, "dist"):
            if mode == "fused" and self.comm.world > 1:
                raise RuntimeError("fused collectives need one CUDA rank per process (torch.distributed / NCCL plumbing)")
            return None
        try:
            from ..parallel.fused import FusedCollectives
            return FusedCollectives(self.comm, self.device)
        except Exception:
            if mode == "fused":
                raise
            return None

    def close(self) -> None:
        """Collective: ordered release of the in-kernel collectives' peer-memory segments (see FusedCollectives.close)."""
        if self.fused is not None:
            self.fused.close()

    def _all_reduce_small(self, t: torch.Tensor, op: str) -> None:
        if self.fused is not None and t.dtype == torch.float32 and t.is_contiguous() and t.numel() * self.comm.world <= 4096:
            self.fused.all_reduce_small(t, op)
        else:
            self.comm.all_reduce(t, op).wait()

    # ================================================================================== run state
    def _alloc_run_state(self) -> None:
        cfg, o, dev, dt = self.cfg, self.opts, self.device, self.dtype
        B, T, C, D, QC, V, L = self.B, self.T, cfg.hidden_size, cfg.intermediate_size, cfg.qkv_channels, cfg.vocab_size, cfg.num_hidden_layers
        Hq, HS = cfg.num_attention_heads, cfg.head_size
        BT = B * T
        z = lambda *shape, dtype=dt: torch.zeros(*shape, dtype=dtype, device=dev)
        q = self.quant
        self.inputs = torch.zeros(B, T, dtype=torch.int32, device=dev)
        self.targets = torch.zeros(B, T, dtype=torch.int32, device=dev)
        self.losses = torch.zeros(B, T, dtype=torch.float32, device=dev)
        self.lse_tok = torch.zeros(B, T, dtype=torch.float32, device=dev)
        self.lse_stats = torch.zeros(2, dtype=torch.float32, device=dev)
        self.group_losses = torch.zeros((T + 511) // 512, dtype=torch.float32, device=dev)
        self.norm_io = torch.zeros(2, dtype=torch.float32, device=dev)
        self.norm_partials = torch.zeros(K.NORM_PARTIALS, dtype=torch.float32, device=dev)
        self.stats = torch.zeros(L, N_SLOTS, 2, dtype=torch.float32, device=dev)
        self.freqs = K.rope_table(T, HS, cfg.rope_theta, dev)

        def per_layer(shared: bool, *shape, dtype=dt):
            if shared:
                t = z(*shape, dtype=dtype)
                return [t] * L
            return [z(*shape, dtype=dtype) for _ in range(L)]

        a = SimpleNamespace()
        a.x = ResidualStore(L + 1, (BT, C), dt, dev, o.offload_residual)     # residual stream entering each layer (+ final)
        a.rstd1 = per_layer(False, BT, dtype=torch.float32)
        a.rstd2 = per_layer(False, BT, dtype=torch.float32)
        a.lse = per_layer(False, B, Hq, T, dtype=torch.float32)
        re_ln1 = o.recompute_rms_norm or o.recompute_att or o.recompute_block
        re_qkv = o.recompute_qkv or o.recompute_att or o.recompute_block
        re_att = o.recompute_att or o.recompute_block
        re_ln2 = o.recompute_rms_norm or o.recompute_ffn or o.recompute_block
        re_up = o.recompute_ffn
        re_sw = o.recompute_swiglu or o.recompute_ffn or o.recompute_block
        self.re = SimpleNamespace(ln1=re_ln1, qkv=re_qkv, att=re_att, ln2=re_ln2, up=re_up, sw=re_sw, block=o.recompute_block)
        # bf16 values of the quantised GEMM inputs are only needed until they are quantised
        a.ln1 = per_layer(re_ln1 or q, BT, C)
        a.ln2 = per_layer(re_ln2 or q, BT, C)
        a.swiglu = per_layer(re_sw or q, BT, D)
        a.qkv = per_layer(re_qkv, B, T, QC // HS, HS)
        a.att = per_layer(re_att, BT, C)
        a.res_att = per_layer(o.recompute_block, BT, C)
        a.up = per_layer(re_up, BT, 2 * D)
        if q:
            a.ln1_q = per_layer(re_ln1, BT, C, dtype=self.qdtype)
            a.ln2_q = per_layer(re_ln2, BT, C, dtype=self.qdtype)
            a.swiglu_q = per_layer(re_sw, BT, D, dtype=self.qdtype)
            a.att_q = per_layer(True, BT, C, dtype=self.qdtype)
        self.acts = a
        self.lnf = z(BT, C)
        self.rstd_f = torch.zeros(BT, dtype=torch.float32, device=dev)
        # ---- temporaries shared by all layers, carved from ONE stack buffer (utils/memory.py, role of the reference's
        # DeviceMemoryStack, stack.cpp:13-56 / llama_model.cpp:899-925).  The allocation pattern of a step is replayed twice:
        # first on a dry-run stack, whose high-water mark sizes the backing buffer, then on the real one.  Buffers of
        # different phases (LM head: logits chunks; block backward: activation gradients, their fp8 copies and transposes)
        # are pushed and popped per phase, so they share addresses; the addresses are the same every step (CUDA graphs).
        from ..utils.memory import DeviceMemoryStack
        chunks = max(1, o.lmhead_chunks)
        if BT % chunks:
            raise ValueError("lmhead_chunks must divide batch * seq_len")
        self._kmajor = bool(q and o.kmajor_backward and dev.type == "cuda" and self.qdtype in F8_TYPES and self.gdtype in F8_TYPES
                            and all(v % 16 == 0 for v in (BT, C, 2 * D, QC)))
        on_gpu = dev.type == "cuda"

        def plan(stack):
            t = SimpleNamespace()
            names = []

            def A(name, *shape, dtype=dt):
                setattr(t, name, stack.allocate(shape, dtype, name))
                names.append(name)

            def end_phase(first, last=None):
                for n in reversed(names[first:last]):
                    stack.free(getattr(t, n))
            # whole step
            A("proj", BT, C)                 # attention-out / mlp-down results, folded into the next residual add
            A("d_res", BT, C)                # gradient of the residual stream
            A("d_ln", BT, C)                 # gradient wrt a norm output / attention output
            A("norm_scratch", K.rmsnorm_backward_scratch_elems(C, dev), dtype=torch.float32)
            A("bias_scratch", 64 * QC, dtype=torch.float32)
            base = len(names)
            # LM-head phase
            A("logits", BT // chunks, V)
            t.logits2 = t.lnf_T = None
            if on_gpu and o.overlap_lmhead and chunks > 1:
                A("logits2", BT // chunks, V)    # the LM-head gradients of a chunk run beside the next chunk's logits + classifier
            t.dlogits_T = None
            if on_gpu:
                A("lnf_T", C, BT // chunks)      # lnf chunk transposed, B operand of the LM-head dW GEMM
                if o.lmhead_transposed_operands and o.lmhead_transpose_dlogits and V % 8 == 0 and (BT // chunks) % 8 == 0:
                    A("dlogits_T", V, BT // chunks)      # d(logits) chunk transposed, A operand of the LM-head dW GEMM
            end_phase(base)
            first = len(names)
            # block-backward phase
            A("d_sw", BT, D)
            A("d_qkv", B, T, QC // HS, HS)
            A("att_scratch", B * Hq * T, dtype=torch.float32)
            if q:
                A("d_res_q", BT, C, dtype=self.gdtype)
                A("d_up_q", BT, 2 * D, dtype=self.gdtype)
                A("d_qkv_q", BT, QC, dtype=self.gdtype)
            # fp8 backward with every GEMM operand K-major: transposed copies of the output gradients (written by the pass
            # that quantises them), of the layer inputs and of the weights (fp8 -> fp8 transposes next to their GEMM)
            t.d_res_qT = t.d_up_qT = t.d_qkv_qT = None
            if self._kmajor:
                A("d_res_qT", C, BT, dtype=self.gdtype)
                A("d_up_qT", 2 * D, BT, dtype=self.gdtype)
                A("d_qkv_qT", QC, BT, dtype=self.gdtype)
                A("inp_qT", max(C, D) * BT, dtype=self.qdtype)
                A("w_T", max(2 * D, QC, C) * max(C, D), dtype=self.qdtype)
            if self.mx:
                # one A-role and one B-role operand buffer (values + tiled scales), sized for the largest use
                feat = max(C, QC, 2 * D)
                a_uses = [(BT, feat), (feat, BT)]
                b_uses = [(2 * D, C), (C, 2 * D), (QC, C), (C, QC), (C, D), (D, C), (C, BT), (D, BT)]
                f8, u8 = torch.float8_e4m3fn, torch.uint8
                A("mx_a_q", BT * feat, dtype=f8)
                A("mx_a_sf", max(K.mx_sf_bytes(r, k, K.MX_TILE_A) for r, k in a_uses), dtype=u8)
                A("mx_a2_q", BT * feat, dtype=f8)                 # column form of an output gradient
                A("mx_a2_sf", max(K.mx_sf_bytes(r, k, K.MX_TILE_A) for r, k in a_uses), dtype=u8)
                A("mx_b2_q", BT * max(C, D), dtype=f8)            # transposed layer input (second stream)
                A("mx_b2_sf", max(K.mx_sf_bytes(r, BT, K.MX_TILE_B) for r in (C, D)), dtype=u8)
                A("mx_b_q", max(r * k for r, k in b_uses), dtype=f8)
                A("mx_b_sf", max(K.mx_sf_bytes(r, k, K.MX_TILE_B) for r, k in b_uses), dtype=u8)
            end_phase(first)
            end_phase(0, base)
            return t

        sizing = DeviceMemoryStack(0, dry_run=True)
        plan(sizing)
        self.stack = DeviceMemoryStack(sizing.high_water, device=dev)
        self.stack.backing.zero_()
        t = plan(self.stack)
        self.stack_report = {"capacity": self.stack.capacity, "high_water": self.stack.high_water, "breakdown": sizing.high_water_breakdown()}
        self.tmp = t
        self.host_scalars = torch.zeros(8, dtype=torch.float32, pin_memory=(dev.type == "cuda"))
        self._submarks = bool(self.opts.trigger_timing_events and os.environ.get("LLMQ_SUBMARKS", "0") == "1")

    # ---- optional phase timing (--debug-time-breakdown): CUDA events on the main stream, read after the step
    def _mark(self, name: str) -> None:
        if self.opts.trigger_timing_events and self.device.type == "cuda":
            ev = torch.cuda.Event(enable_timing=True)
            ev.record(torch.cuda.current_stream(self.device))
            self._marks.append((name, ev))

    def _submark(self, name: str) -> None:
        """Finer marks inside the blocks (LLMQ_SUBMARKS=1, plain launches only): the phase totals then cover only their tails."""
        if self._submarks and self.graphs is None:
            self._mark(name)

    def time_breakdown(self) -> Dict[str, float]:
        """Milliseconds per phase since the last call (phases of all micro-steps are summed); synchronises."""
        marks, self._marks = self._marks, []
        out: Dict[str, float] = {}
        if len(marks) < 2:
            return out
        marks[-1][1].synchronize()
        for (n0, e0), (n1, e1) in zip(marks[:-1], marks[1:]):
            if n1 != "start":
                out[n1] = out.get(n1, 0.0) + e0.elapsed_time(e1)
        return out

    def abs_maxes(self) -> Dict[str, List[float]]:
        """Abs-max of every quantised activation / gradient slot, per layer (--debug-log-abs-max)."""
        vals = self.stats[:, :, 0].float().cpu()
        return {f"layer{l}": [round(float(v), 6) for v in vals[l]] for l in range(vals.shape[0])}

    def _slot(self, l: int, s: int):
        st = self.stats[l, s]
        return st[0:1], st[1:2]

    # ================================================================================== init / import
    def init_weights(self, seed: int = 42) -> None:
        """N(0, 0.02) for qkv / up / embeddings / head, N(0, 0.02/sqrt(2L)) for the two output projections,
        ones for norms, zeros for biases.  The stream of a tensor depends only on (seed, tensor index) and the
        element index, so every world size produces the same model."""
        w = self.weights
        for idx, (name, master, spec, l) in enumerate(w.master_items()):
            rows_per = master.shape[0]
            offset = self.comm.rank * rows_per * (master.numel() // max(rows_per, 1))
            dev_t = master if master.device.type == self.device.type else torch.empty(master.shape, dtype=master.dtype, device=self.device)
            if spec.init_std < 0:
                dev_t.fill_(1.0)
            elif spec.init_std == 0:
                dev_t.zero_()
            else:
                K.fill_normal(dev_t, 0.0, spec.init_std, seed, subsequence=idx, offset=offset)
            if dev_t is not master:
                master.copy_(dev_t)
        self.on_weights_changed()

    def on_weights_changed(self) -> None:
        """After init / import / checkpoint restore: refresh abs-max values and invalidate the work copies."""
        self.weights.sync_absmax(recompute=True)
        self.weights.invalidate()

    # ================================================================================== quantised matmuls
    def _mx_gemm(self, out, a, b, *, a_t=False, b_t=False, bias=None, accumulate=False):
        """out (+)= op(a) @ op(b)^T with block-scaled e4m3 copies of both operands; ``a_t`` / ``b_t`` contract over the rows
        of the stored matrix (quantised along the rows, used transposed)."""
        t = self.tmp
        a, b = a.reshape(-1, a.shape[-1]), b.reshape(-1, b.shape[-1])
        ra, ka = (a.shape[1], a.shape[0]) if a_t else a.shape
        rb, kb = (b.shape[1], b.shape[0]) if b_t else b.shape
        aq, bq = t.mx_a_q[:ra * ka].view(ra, ka), t.mx_b_q[:rb * kb].view(rb, kb)
        K.quantize_mx(a, transpose=a_t, operand="a", q_out=aq, sf_out=t.mx_a_sf)
        K.quantize_mx(b, transpose=b_t, operand="b", q_out=bq, sf_out=t.mx_b_sf)
        K.gemm_mx(out.reshape(-1, out.shape[-1]), aq, t.mx_a_sf, bq, t.mx_b_sf, bias=bias, accumulate=accumulate)

    def _fwd_mm(self, out, act, act_q, slot, W, w_scale, bias=None, ready=None):
        if self.mx:
            self._mx_gemm(out, act, W, bias=bias)
            return
        if not self.quant:
            K.gemm(out, act, W, bias=bias, ready=ready)
            return
        am, sc = slot
        if act is not None:
            K.quantize(act_q, sc, act, am)
        K.gemm(out, act_q, W, bias=bias, scale_a=sc, scale_b=w_scale, ready=ready)

    def _bwd_mm(self, dinp, dW, dbias, dout, dout_q, slot, inp, inp_q, inp_scale, W, w_scale, accumulate, ready=None, dw_rs=None,
                swiglu_inout=None, swiglu_absmax=None, dout_qT=None, inp_qT_ready=False, dout_ready=False, before_dw=None):
        """dinp = dout @ W;  dW (+)= dout^T @ inp;  dbias += colsum(dout).  Operands are read in place:
        W is the MN-major B operand of the first product, dout and inp the MN-major operands of the second.
        ``dw_rs`` (from ``GradientManager.fused_dw``) runs the weight-gradient GEMM with its reduce-scatter inside.
        ``swiglu_inout`` ([up | gate] -> [d_up | d_gate], in place): the input-gradient GEMM applies the SwiGLU backward
        in its epilogue instead of writing ``dinp``.  ``dout_ready``: ``dout_q`` / ``dout_qT`` and the scale already hold the
        quantised gradient (``dout`` itself is not read).  ``before_dw`` runs on the main stream between the input-gradient
        GEMM and the launch of the weight-gradient GEMM (K-major fp8 path only)."""
        if self.mx:
            # dout feeds two GEMMs with different contraction axes: its row form and its column form come from one pass
            t = self.tmp
            d2 = dout.reshape(-1, dout.shape[-1])
            BT, OC = d2.shape
            d_rows, d_cols = t.mx_a_q[:BT * OC].view(BT, OC), t.mx_a2_q[:BT * OC].view(OC, BT)
            # d_cols and the transposed input are read by the weight-gradient GEMM on the second stream: the previous one
            # must have finished with those buffers before they are rewritten
            self._wait_dw(self._mx_dw_event)
            if dinp is not None:
                K.quantize_mx_both(d2, q_rows=d_rows, sf_rows=t.mx_a_sf, q_cols=d_cols, sf_cols=t.mx_a2_sf)
                wq = t.mx_b_q[:W.numel()].view(W.shape[1], W.shape[0])
                K.quantize_mx(W, transpose=True, operand="b", q_out=wq, sf_out=t.mx_b_sf)
                K.gemm_mx(dinp.reshape(BT, -1), d_rows, t.mx_a_sf, wq, t.mx_b_sf)
            else:
                K.quantize_mx(d2, transpose=True, operand="a", q_out=d_cols, sf_out=t.mx_a2_sf)
            i2 = inp.reshape(BT, -1)
            iq = t.mx_b2_q[:i2.numel()].view(i2.shape[1], BT)

            def dw():
                K.quantize_mx(i2, transpose=True, operand="b", q_out=iq, sf_out=t.mx_b2_sf)
                K.gemm_mx(dW, d_cols, t.mx_a2_sf, iq, t.mx_b2_sf, accumulate=accumulate)
            self._mx_dw_event = self._launch_dw(dw)
            if dbias is not None:
                K.bias_backward(dbias, dout, self.tmp.bias_scratch, accumulate=True)
            return
        if not self.quant:
            if swiglu_inout is not None:
                K.gemm_swiglu_backward(swiglu_inout, dout, W, absmax=swiglu_absmax)
            elif dinp is not None:
                K.gemm(dinp, dout, W, b_mn=True, ready=ready)
            if dw_rs is not None:
                self._launch_dw(lambda: dw_rs(dout, inp))
            else:
                self._launch_dw(lambda: K.gemm(dW, dout, inp, a_mn=True, b_mn=True, accumulate=accumulate))
            if dbias is not None:
                K.bias_backward(dbias, dout, self.tmp.bias_scratch, accumulate=True)
            return
        am, sc = slot
        t = self.tmp
        kmajor = self._kmajor and dout_qT is not None and ready is None
        assert kmajor or (not dout_ready and before_dw is None)
        if dout_ready:
            pass
        elif kmajor:
            K.quantize_transpose(dout_q, dout_qT, sc, dout, am)
        else:
            K.quantize(dout_q, sc, dout, am)
        if swiglu_inout is not None:
            K.gemm_swiglu_backward(swiglu_inout, dout_q, W, scale_a=sc, scale_b=w_scale, absmax=swiglu_absmax)
        elif dinp is not None:
            if kmajor:
                WT = t.w_T[:W.numel()].view(W.shape[1], W.shape[0])
                K.transpose(WT, W)
                K.gemm(dinp, dout_q, WT, scale_a=sc, scale_b=w_scale)
            else:
                K.gemm(dinp, dout_q, W, b_mn=True, scale_a=sc, scale_b=w_scale, ready=ready)
        if kmajor:
            if before_dw is not None:
                before_dw()
            i2 = inp_q.reshape(-1, inp_q.shape[-1])
            iT = t.inp_qT[:i2.numel()].view(i2.shape[1], i2.shape[0])

            have_T = inp_qT_ready

            def dw():
                # the side stream runs these two in order, so one transposed-input buffer serves every GEMM of the block
                if not have_T:
                    K.transpose(iT, i2)
                if dw_rs is not None:
                    dw_rs(dout_qT, iT, sc, inp_scale, a_mn=False, b_mn=False)
                else:
                    K.gemm(dW, dout_qT, iT, scale_a=sc, scale_b=inp_scale, accumulate=accumulate)
            self._launch_dw(dw)
        elif dw_rs is not None:
            self._launch_dw(lambda: dw_rs(dout_q, inp_q, sc, inp_scale))
        else:
            self._launch_dw(lambda: K.gemm(dW, dout_q, inp_q, a_mn=True, b_mn=True, scale_a=sc, scale_b=inp_scale, accumulate=accumulate))
        if dbias is not None:
            K.bias_backward(dbias, dout_q, self.tmp.bias_scratch, scale_a=sc, accumulate=True)

    # ---- weight-gradient GEMMs off the critical path
    # A dW GEMM only feeds the optimizer, while the chain dX GEMM -> element-wise kernels -> next dX GEMM decides the
    # length of the backward pass.  On the GPU the dW GEMMs therefore go to a second, higher-priority stream: their
    # CTAs (one per SM, tensor-core bound) share the SMs with the memory-bound element-wise kernels of the main
    # stream.  Every block joins the side stream before it ends, so nothing outlives the buffers it reads.
    def _launch_dw(self, fn, stream=None):
        side = stream if stream is not None else self._dw_stream
        if side is None:
            fn()
            return None
        main = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(main)
        with torch.cuda.stream(side):
            side.wait_event(ready)
            fn()
            done = torch.cuda.Event()
            done.record(side)
        self._dw_events.append(done)
        return done

    def _wait_dw(self, ev) -> None:
        """The main stream waits for one weight-gradient GEMM."""
        if ev is not None:
            torch.cuda.current_stream(self.device).wait_event(ev)

    def _join_dw(self) -> None:
        """The main stream waits for every outstanding weight-gradient GEMM."""
        if not self._dw_events:
            return
        main = torch.cuda.current_stream(self.device)
        for e in self._dw_events:
            main.wait_event(e)
        self._dw_events = []
        self._mx_dw_event = None

    # ================================================================================== forward
    def forward(self, inputs: torch.Tensor, micro_step: int = 0) -> None:
        """inputs: int32 (B, T) on any device.  Activations stay in the run state for ``backward``."""
        cfg, a, w = self.cfg, self.acts, self.weights
        L = cfg.num_hidden_layers
        self._mark("start")
        r_fwd = nvtx.push("forward", self.device)
        if inputs is not None:                    # None: the caller already placed the tokens in self.inputs
            self.inputs.copy_(inputs.reshape(self.B, self.T), non_blocking=True)
        K.encoder_forward(a.x.write_target(0), self.inputs, w.get_embeddings())
        a.x.written(0)
        self.stats.zero_()
        w.gather_block(0)
        split = self._split_blocks
        for l in range(L):
            if l + 1 < L and not split:
                w.gather_block(l + 1)
            r_layer = nvtx.push(f"Layer {l}", self.device)
            p = w.get_block(l)
            self._submark("f:wait")
            am, _ = self._slot(l, S_LN1)
            if l == 0:
                K.rmsnorm_forward(a.ln1[l], a.rstd1[l], a.x.current(0), p.ln1_w, cfg.rms_norm_eps, absmax=am)
            else:
                K.rmsnorm_forward(a.ln1[l], a.rstd1[l], a.res_att[l - 1], p.ln1_w, cfg.rms_norm_eps, residual_out=a.x.write_target(l),
                                  inp2=self.tmp.proj, absmax=am)
                a.x.written(l)
            self._submark("f:ln1")
            if split:
                # The gather of the next block starts behind this block's first GEMM, so that its pushes (a grid over all SMs)
                # share the GPU with RoPE and attention, whose many short CTAs flow around them, instead of holding up the
                # CTA pairs of a persistent GEMM: started at the top of the block they delayed the QKV GEMM by their own length.
                self._run_block(("fwd", l, 0), lambda: self._forward_block(l, p, 0))
                if l + 1 < L:
                    w.gather_block(l + 1)
                self._run_block(("fwd", l, 1), lambda: self._forward_block(l, p, 1))
            else:
                self._run_block(("fwd", l), lambda: self._forward_block(l, p))
            w.release_block(l)
            nvtx.pop(r_layer)
        K.rmsnorm_forward(self.lnf, self.rstd_f, a.res_att[L - 1], w.get_lnf(), cfg.rms_norm_eps, residual_out=a.x.write_target(L),
                          inp2=self.tmp.proj)
        a.x.written(L)
        nvtx.pop(r_fwd)

    def _run_block(self, key: tuple, fn) -> None:
        if self.graphs is not None:
            self.graphs.run(key, fn)
        else:
            fn()

    def _forward_block(self, l: int, p, part: Optional[int] = None) -> None:
        """``part``: None = the whole block, 0 = the QKV projection only, 1 = everything behind it."""
        cfg, a, t = self.cfg, self.acts, self.tmp
        Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        BT = self.B * self.T
        if part != 1:
            qkv2d = a.qkv[l].view(BT, cfg.qkv_channels)
            self._fwd_mm(qkv2d, a.ln1[l], a.ln1_q[l] if self.quant else None, self._slot(l, S_LN1), p.qkv_w, p.scales["qkv_w"], p.qkv_b, ready=p.ready["qkv_w"])
            self._submark("f:qkv")
        if part == 0:
            return
        K.rope(a.qkv[l], a.qkv[l], self.freqs, Hq, Hkv)
        att4 = a.att[l].view(self.B, self.T, Hq, cfg.head_size)
        K.attention_forward(att4, a.lse[l], a.qkv[l], Hq, Hkv, absmax=self._slot(l, S_ATT)[0] if self.quant else None)
        self._submark("f:att")
        self._fwd_mm(t.proj, a.att[l], a.att_q[l] if self.quant else None, self._slot(l, S_ATT), p.o_w, p.scales["o_w"], ready=p.ready["o_w"])
        self._submark("f:o")
        K.rmsnorm_forward(a.ln2[l], a.rstd2[l], a.x.current(l), p.ln2_w, cfg.rms_norm_eps, residual_out=a.res_att[l], inp2=t.proj,
                          absmax=self._slot(l, S_LN2)[0])
        self._submark("f:ln2")
        if self._fuse_swiglu and (int(self.opts.fuse_swiglu) & 1) and p.ready["up_w"] is None:
            # up projection and SwiGLU from one accumulator tile: the activation never re-reads the projection
            am, sc = self._slot(l, S_LN2)
            if self.quant:
                K.quantize(a.ln2_q[l], sc, a.ln2[l], am)
                K.gemm_swiglu_forward(a.up[l], a.swiglu[l], a.ln2_q[l], p.up_w, scale_a=sc, scale_b=p.scales["up_w"],
                                      absmax=self._slot(l, S_SWIGLU)[0])
            else:
                K.gemm_swiglu_forward(a.up[l], a.swiglu[l], a.ln2[l], p.up_w, absmax=self._slot(l, S_SWIGLU)[0])
        else:
            self._fwd_mm(a.up[l], a.ln2[l], a.ln2_q[l] if self.quant else None, self._slot(l, S_LN2), p.up_w, p.scales["up_w"], ready=p.ready["up_w"])
            self._submark("f:up")
            K.swiglu_forward(a.swiglu[l], a.up[l], absmax=self._slot(l, S_SWIGLU)[0])
            self._submark("f:swiglu")
        self._fwd_mm(t.proj, a.swiglu[l], a.swiglu_q[l] if self.quant else None, self._slot(l, S_SWIGLU), p.down_w, p.scales["down_w"], ready=p.ready["down_w"])
        self._submark("f:down")

    # ================================================================================== validation
    @torch.no_grad()
    def validate(self, inputs: torch.Tensor, targets: torch.Tensor):
        """Returns (mean loss, mean loss over the first 1024 positions) of one batch, averaged over ranks."""
        with nvtx.range("validate", self.device):
            self.forward(inputs)
            self.targets.copy_(targets.reshape(self.B, self.T), non_blocking=True)
            self.losses.zero_()
            with nvtx.range("lm-head", self.device):
                self._lmhead(write_grads=False, dloss=0.0, z_loss=0.0, accumulate_dw=False)
            return self._reduce_loss(None)

    def _reduce_loss(self, positions_per_rank: Optional[float]):
        """Mean loss and mean loss over the first 1024 positions.  ``positions_per_rank`` is the number of
        target positions behind ``self.losses`` on each rank (None: count the unmasked targets)."""
        K.grouped_loss_sum(self.group_losses, self.losses)
        gl = self.group_losses.clone()
        if positions_per_rank is None:
            cnt = (self.targets != -100).sum().float().reshape(1)
            if self.comm.world > 1:
                self._all_reduce_small(cnt, "avg")
        else:
            cnt = torch.full((1,), float(positions_per_rank), device=self.device)
        if self.comm.world > 1:
            self._all_reduce_small(gl, "avg")
        cnt = cnt.clamp_min(1)
        total = gl.sum() / cnt
        n1k = min(self.T, 1024)
        first = gl[: (n1k + 511) // 512].sum() / (cnt * n1k / self.T)
        return float(total.item()), float(first.item())

    # ================================================================================== LM head
    def _lmhead(self, write_grads: bool, dloss: float, z_loss: float, accumulate_dw: bool) -> None:
        cfg, t = self.cfg, self.tmp
        BT, C, V = self.B * self.T, cfg.hidden_size, cfg.vocab_size
        chunks = max(1, self.opts.lmhead_chunks)
        n = BT // chunks
        W = self.weights.get_head()
        head_name = "embed" if cfg.tie_word_embeddings else "lm_head"
        dW = self.grads.nb_full[head_name] if write_grads else None
        tg = self.targets.view(BT)
        losses, lse = self.losses.view(BT), self.lse_tok.view(BT)
        # The backward GEMMs read W and lnf as B operands along the "wrong" axis; with MN-major TMA loads they run at
        # 0.6-0.8 of the K-major rate, so on the GPU the two small transposes below (W^T once per optimizer step,
        # lnf^T per chunk) are cheaper than letting the GEMM read them in place.
        use_t = write_grads and W.is_cuda and self.opts.lmhead_transposed_operands
        WT = self._head_transposed(W) if use_t else None
        # The chain is logits GEMM -> classifier -> next chunk's logits GEMM; dW and dX of a chunk only need its
        # classifier, so with a second logits buffer they run on the side stream under the next chunk's classifier.
        side = self._side_stream if (write_grads and t.logits2 is not None and self.opts.overlap_lmhead) else None
        main = torch.cuda.current_stream(self.device) if side is not None else None
        busy = [None, None]                                     # side-stream event of the last reader of each logits buffer
        for c in range(chunks):
            sl = slice(c * n, (c + 1) * n)
            logits = t.logits if (side is None or c % 2 == 0) else t.logits2
            if side is not None and busy[c % 2] is not None:
                main.wait_event(busy[c % 2])
            K.gemm(logits, self.lnf[sl], W)
            K.fused_classifier(logits, losses[sl], lse[sl], tg[sl], dloss, z_reg=z_loss * dloss, write_dlogits=write_grads)
            if not write_grads:
                continue

            def grads_of_chunk(logits=logits, sl=sl, c=c):
                if use_t:
                    K.transpose(t.lnf_T, self.lnf[sl])
                    K.gemm(t.d_ln[sl], logits, WT)
                    if t.dlogits_T is not None:
                        K.transpose(t.dlogits_T, logits)            # both operands of dW K-major
                        K.gemm(dW, t.dlogits_T, t.lnf_T, accumulate=accumulate_dw or c > 0)
                    else:
                        K.gemm(dW, logits, t.lnf_T, a_mn=True, accumulate=accumulate_dw or c > 0)
                else:
                    K.gemm(dW, logits, self.lnf[sl], a_mn=True, b_mn=True, accumulate=accumulate_dw or c > 0)
                    K.gemm(t.d_ln[sl], logits, W, b_mn=True)

            if side is None:
                grads_of_chunk()
            else:
                busy[c % 2] = self._launch_dw(grads_of_chunk, side)
        self._join_dw()
        if write_grads and not cfg.tie_word_embeddings:
            self.grads.notify_non_block(head_name)
        # max and sum of the per-token log-sum-exp over ALL micro-steps of the optimizer step (llama_model.cpp accumulates them too)
        K.lse_stats(self.lse_stats, self.lse_tok.view(-1), accumulate=accumulate_dw)

    def _head_transposed(self, W: torch.Tensor) -> torch.Tensor:
        """W^T (C, V) of the LM-head weight, refreshed when the weights changed (once per optimizer step)."""
        ver = (self.weights.version, W.data_ptr())
        if getattr(self, "_head_T", None) is None:
            self._head_T = torch.empty(W.shape[1], W.shape[0], dtype=W.dtype, device=W.device)
            self._head_T_ver = None
        if self._head_T_ver != ver:
            K.transpose(self._head_T, W)
            self._head_T_ver = ver
        return self._head_T

    # ================================================================================== backward
    def backward(self, inputs: torch.Tensor, targets: torch.Tensor, z_loss: float = 0.0, grad_accum: int = 1,
                 micro_step: int = 0) -> None:
        cfg, a, t, w, g = self.cfg, self.acts, self.tmp, self.weights, self.grads
        L, C = cfg.num_hidden_layers, cfg.hidden_size
        if targets is not None:
            self.targets.copy_(targets.reshape(self.B, self.T), non_blocking=True)
        if micro_step == 0:
            g.begin_step()
            self.losses.zero_()
        g.start_micro_step(micro_step, grad_accum)
        dloss = 1.0 / (self.B * self.T * grad_accum)
        self._mark("forward")
        r_bwd = nvtx.push("backward", self.device)
        with nvtx.range("lm-head", self.device):
            self._lmhead(write_grads=True, dloss=dloss, z_loss=z_loss, accumulate_dw=micro_step > 0)
        self._mark("lm-head")
        # final norm: t.d_ln holds d(lnf); produce d(residual stream) in t.d_res
        t.d_res.zero_()
        K.rmsnorm_backward(t.d_res, g.nb_full["lnf_w"], t.norm_scratch, t.d_ln, a.x.get(L), w.get_lnf(), self.rstd_f,
                           absmax=self._slot(L - 1, S_DRESFFN)[0], accumulate_dweight=True)
        g.notify_non_block("lnf_w")
        w.gather_block(L - 1)
        for l in range(L - 1, -1, -1):
            r_layer = nvtx.push(f"Layer {l}", self.device)
            dw, acc = g.get_block_full(l)
            a.x.prefetch(l - 1)
            split = self._split_blocks
            if l > 0 and not split:
                w.gather_block(l - 1)
            p = w.get_block(l)
            self._submark("b:wait")

            def body(part, l=l, p=p, dw=dw, acc=acc):
                if part != 1:
                    self._recompute_block(l, p)
                    self._submark("b:recompute")
                self._backward_block(l, p, dw, acc, part)
            if split:
                # as in forward(): the next gather starts behind the MLP and output-projection GEMMs, beside the attention kernels
                self._run_block(("bwd", l, bool(acc), 0), lambda: body(0))
                if l > 0:
                    w.gather_block(l - 1)
                self._run_block(("bwd", l, bool(acc), 1), lambda: body(1))
            else:
                self._run_block(("bwd", l, bool(acc)), lambda: body(None))
            # LN1 backward adds into the residual gradient, which then belongs to layer l-1 (or the embedding)
            slot = self._slot(l - 1, S_DRESFFN)[0] if l > 0 else None
            K.rmsnorm_backward(t.d_res, dw["ln1_w"], t.norm_scratch, t.d_ln, a.x.get(l), p.ln1_w, a.rstd1[l], absmax=slot,
                               accumulate_dweight=True)
            self._submark("b:ln1")
            w.release_block(l)
            g.notify_block(l)
            self._submark("b:notify")
            nvtx.pop(r_layer)
        if not cfg.tie_word_embeddings and micro_step == 0:
            g.nb_full["embed"].zero_()             # untied: nothing has written this buffer yet in this step
        K.encoder_backward(g.nb_full["embed"], t.d_res, self.inputs)
        g.notify_non_block("embed")
        g.end_micro_step()
        nvtx.pop(r_bwd)
        self._mark("backward")

    def _recompute_block(self, l: int, p) -> None:
        cfg, a, t, re = self.cfg, self.acts, self.tmp, self.re
        Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        BT = self.B * self.T
        q = self.quant

        def renorm(y, yq, slot_id, x, wt, rstd):
            am, sc = self._slot(l, slot_id)
            if q:
                K.rmsnorm_forward(None, None, x, wt, cfg.rms_norm_eps, q_out=yq, known_absmax=am, q_scale=sc)
            else:
                K.rmsnorm_forward(y, None, x, wt, cfg.rms_norm_eps)

        if re.ln1:
            renorm(a.ln1[l], a.ln1_q[l] if q else None, S_LN1, a.x.get(l), p.ln1_w, a.rstd1[l])
        if re.qkv:
            qkv2d = a.qkv[l].view(BT, cfg.qkv_channels)
            self._fwd_mm(qkv2d, None if q else a.ln1[l], a.ln1_q[l] if q else None, self._slot(l, S_LN1), p.qkv_w, p.scales["qkv_w"], p.qkv_b, ready=p.ready["qkv_w"])
            if not q:
                pass
            K.rope(a.qkv[l], a.qkv[l], self.freqs, Hq, Hkv)
        if re.att:
            K.attention_forward(a.att[l].view(self.B, self.T, Hq, cfg.head_size), a.lse[l], a.qkv[l], Hq, Hkv)
        if q:
            # the fp8 copy of the attention output lives in a buffer shared by all layers
            am, sc = self._slot(l, S_ATT)
            K.quantize(a.att_q[l], sc, a.att[l], am)
        if re.block:
            self._fwd_mm(t.proj, None if q else a.att[l], a.att_q[l] if q else None, self._slot(l, S_ATT), p.o_w, p.scales["o_w"], ready=p.ready["o_w"])
            am, sc = self._slot(l, S_LN2)
            if q:
                K.rmsnorm_forward(None, None, a.x.get(l), p.ln2_w, cfg.rms_norm_eps, residual_out=a.res_att[l], inp2=t.proj,
                                  q_out=a.ln2_q[l], known_absmax=am, q_scale=sc)
            else:
                K.rmsnorm_forward(a.ln2[l], None, a.x.get(l), p.ln2_w, cfg.rms_norm_eps, residual_out=a.res_att[l], inp2=t.proj)
        elif re.ln2:
            renorm(a.ln2[l], a.ln2_q[l] if q else None, S_LN2, a.res_att[l], p.ln2_w, a.rstd2[l])
        if re.up:
            self._fwd_mm(a.up[l], None if q else a.ln2[l], a.ln2_q[l] if q else None, self._slot(l, S_LN2), p.up_w, p.scales["up_w"], ready=p.ready["up_w"])
        self._swiglu_T_ready = False
        if re.sw:
            am, sc = self._slot(l, S_SWIGLU)
            if self._swiglu_two_pass(p):
                pass        # the first pass of the SwiGLU backward writes the transposed activation (see _backward_block)
            elif q and self._kmajor and self.qdtype == torch.float8_e4m3fn and self.dtype == torch.bfloat16 and self.grads_use_kmajor_dw():
                # the recomputed activation only feeds the down projection's weight-gradient GEMM, which reads it
                # transposed: write just that copy (into the transposed-input buffer the GEMM reads next)
                D = cfg.intermediate_size
                K.swiglu_forward_transposed(t.inp_qT[:D * BT].view(D, BT), a.up[l], known_absmax=am, q_scale=sc)
                self._swiglu_T_ready = True
            elif q:
                K.swiglu_forward(None, a.up[l], q_out=a.swiglu_q[l], known_absmax=am, q_scale=sc)
            else:
                K.swiglu_forward(a.swiglu[l], a.up[l])

    def grads_use_kmajor_dw(self) -> bool:
        """True when the weight-gradient GEMMs of the blocks take the K-major path of ``_bwd_mm`` (no in-GEMM flag polling)."""
        return self._kmajor and os.environ.get("LLMQ_GEMM_POLL", "0") != "1"

    def _swiglu_two_pass(self, p) -> bool:
        """True when the SwiGLU backward runs as abs-max pass + quantising pass (``K.swiglu_backward_stats`` /
        ``K.swiglu_backward_quant``): e4m3 GEMMs on K-major operands are the only readers of [d_up | d_gate], so its bf16
        form is never written, and the first pass doubles as the SwiGLU recompute for the down projection's dW GEMM."""
        e4 = torch.float8_e4m3fn
        return bool(self.quant and self._kmajor and self.opts.swiglu_backward_two_pass and self.qdtype == e4 and self.gdtype == e4
                    and self.dtype == torch.bfloat16 and self.grads_use_kmajor_dw()
                    and p.ready["down_w"] is None and p.ready["up_w"] is None
                    and not (self._fuse_swiglu and int(self.opts.fuse_swiglu) & 2))

    def _backward_block(self, l: int, p, dw: Dict[str, torch.Tensor], acc: bool, part: Optional[int] = None) -> None:
        """``part``: None = the whole block, 0 = MLP and attention output projection, 1 = attention core and QKV projection."""
        cfg, a, t = self.cfg, self.acts, self.tmp
        Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        BT, q = self.B * self.T, self.quant
        sc_of = lambda s: self._slot(l, s)[1]
        fused_dw = getattr(self.grads, "fused_dw", None)
        rs = (lambda name: fused_dw(l, name)) if (fused_dw is not None and not self.mx) else (lambda name: None)
        if part == 1:
            self._backward_block_attention(l, p, dw, acc, rs, sc_of)
            return
        # ---- MLP down:  d_sw = d_res @ Wdown ; dWdown += d_res^T @ swiglu
        fuse_sw = self._fuse_swiglu and bool(int(self.opts.fuse_swiglu) & 2) and p.ready["down_w"] is None
        two_pass = self._swiglu_two_pass(p)
        sw_T_ready = getattr(self, "_swiglu_T_ready", False)
        before_dw = None
        if two_pass:
            D = cfg.intermediate_size
            # the transposed SwiGLU output for dW(down) comes out of the first pass when the recompute left it to us
            need_act = self.re.sw and not sw_T_ready
            am_sw, sc_sw = self._slot(l, S_SWIGLU)

            def before_dw():
                K.swiglu_backward_stats(self._slot(l, S_DMLPUP)[0], t.d_sw, a.up[l], act_t=t.inp_qT[:D * BT].view(D, BT) if need_act else None,
                                        act_absmax=am_sw if need_act else None, act_scale=sc_sw if need_act else None)
            sw_T_ready = sw_T_ready or need_act
        self._bwd_mm(t.d_sw, dw["down_w"], None, t.d_res, t.d_res_q if q else None, self._slot(l, S_DRESFFN),
                     a.swiglu[l], a.swiglu_q[l] if q else None, sc_of(S_SWIGLU), p.down_w, p.scales["down_w"], acc, ready=p.ready["down_w"], dw_rs=rs("down_w"),
                     swiglu_inout=a.up[l] if fuse_sw else None, swiglu_absmax=self._slot(l, S_DMLPUP)[0], dout_qT=t.d_res_qT,
                     inp_qT_ready=sw_T_ready, before_dw=before_dw)
        self._submark("b:down")
        ev_down = self._dw_events[-1] if self._dw_events else None      # dW(down) reads d_res / its fp8 copy
        # ---- SwiGLU backward, in place over the saved up-projection (unless the GEMM epilogue above already did it)
        if two_pass:
            K.swiglu_backward_quant(t.d_up_q, t.d_up_qT, self._slot(l, S_DMLPUP)[1], t.d_sw, a.up[l], self._slot(l, S_DMLPUP)[0])
        elif not fuse_sw:
            K.swiglu_backward(a.up[l], t.d_sw, a.up[l], absmax=self._slot(l, S_DMLPUP)[0])
        self._submark("b:swiglu")
        # ---- MLP up:  d_ln2 = d_up @ Wup ; dWup += d_up^T @ ln2
        self._bwd_mm(t.d_ln, dw["up_w"], None, a.up[l], t.d_up_q if q else None, self._slot(l, S_DMLPUP),
                     a.ln2[l], a.ln2_q[l] if q else None, sc_of(S_LN2), p.up_w, p.scales["up_w"], acc, ready=p.ready["up_w"], dw_rs=rs("up_w"),
                     dout_qT=t.d_up_qT, dout_ready=two_pass)
        self._submark("b:up")
        # ---- LN2 backward: d_res += ...   (d_res now is the gradient wrt the post-attention residual)
        self._wait_dw(ev_down)                                          # the next two kernels overwrite d_res and its fp8 copy
        K.rmsnorm_backward(t.d_res, dw["ln2_w"], t.norm_scratch, t.d_ln, a.res_att[l], p.ln2_w, a.rstd2[l],
                           absmax=self._slot(l, S_DRESATT)[0], accumulate_dweight=True)
        self._submark("b:ln2")
        # ---- attention out projection
        self._bwd_mm(t.d_ln, dw["o_w"], None, t.d_res, t.d_res_q if q else None, self._slot(l, S_DRESATT),
                     a.att[l], a.att_q[l] if q else None, sc_of(S_ATT), p.o_w, p.scales["o_w"], acc, ready=p.ready["o_w"], dw_rs=rs("o_w"),
                     dout_qT=t.d_res_qT)
        self._submark("b:o")
        if part == 0:
            self._join_dw()
            return
        self._backward_block_attention(l, p, dw, acc, rs, sc_of)

    def _backward_block_attention(self, l: int, p, dw: Dict[str, torch.Tensor], acc: bool, rs, sc_of) -> None:
        cfg, a, t = self.cfg, self.acts, self.tmp
        Hq, Hkv = cfg.num_attention_heads, cfg.num_key_value_heads
        BT, q = self.B * self.T, self.quant
        # ---- attention core
        att4 = a.att[l].view(self.B, self.T, Hq, cfg.head_size)
        K.attention_backward(t.d_qkv, t.att_scratch, t.d_ln.view(self.B, self.T, Hq, cfg.head_size), att4, a.lse[l], a.qkv[l], Hq, Hkv)
        K.rope(t.d_qkv, t.d_qkv, self.freqs, Hq, Hkv, backward=True, absmax=self._slot(l, S_DQKV)[0])
        self._submark("b:att")
        # ---- QKV projection
        dqkv2d = t.d_qkv.view(BT, cfg.qkv_channels)
        self._bwd_mm(t.d_ln, dw["qkv_w"], dw.get("qkv_b"), dqkv2d, t.d_qkv_q if q else None, self._slot(l, S_DQKV),
                     a.ln1[l], a.ln1_q[l] if q else None, sc_of(S_LN1), p.qkv_w, p.scales["qkv_w"], acc, ready=p.ready["qkv_w"], dw_rs=rs("qkv_w"),
                     dout_qT=t.d_qkv_qT)
        self._join_dw()                                                 # the caller reuses d_res, d_ln and the gradient buffers

    # ================================================================================== optimizer
    def update(self, lr: float, beta1: float = 0.9, beta2: float = 0.95, step: int = 1, eps: float = 1e-8,
               weight_decay: float = 0.1, grad_clip: float = 1.0, grad_accum: int = 1) -> Dict[str, float]:
        """Clips by the global norm, applies AdamW to the local shards, returns {loss, loss_1k, norm, z_max, z_mean}."""
        w, g, o = self.weights, self.grads, self.opt_state
        r_upd = nvtx.push("update", self.device)
        g.wait_all()
        # ---- global gradient norm over the local shards
        self.norm_partials.zero_()
        shard_of = {}
        norm_fused = getattr(g, "norm_fused", False)       # the reduce-scatter kernels already summed the squares
        items = list(w.master_items())
        for name, master, spec, l in items:
            shard_of[name] = g.get_block_shard(l)[spec.name] if l is not None else g.get_nb_shard(spec.name)
        # Nothing offloaded: every launch of the norm and AdamW loops has the same arguments each step (the step's scalars
        # travel through device memory), so with --use-cuda-graphs the ~400 small launches become two graph replays.
        on_device = self.device.type == "cuda" and all(
            t.device.type == "cuda" for name, master, spec, l in items for t in (master, shard_of[name], o.m[name], o.v[name]))
        graph_opt = self.graphs is not None and on_device

        def norms():
            for name, master, spec, l in items:
                gs = shard_of[name]
                gd = gs if gs.device.type == self.device.type else gs.to(self.device, non_blocking=True)
                K.norm_squared(self.norm_partials, gd)
        if not norm_fused:
            if graph_opt:
                self.graphs.run(("opt-norm",), norms)
            else:
                norms()
        K.deterministic_sum(self.norm_io[0:1], g.norm_partials if norm_fused else self.norm_partials)
        if self.comm.world > 1:
            self._all_reduce_small(self.norm_io[0:1], "sum")
        K.norm_finish(self.norm_io, grad_clip)
        scale = self.norm_io[1:2]
        # ---- AdamW on every shard
        w.zero_absmax()
        seed_base = (self.rng_state * 1000003) & 0x7FFFFFFF
        if graph_opt:
            if getattr(self, "_opt_hyper", None) is None:
                self._opt_hyper = torch.zeros(8, dtype=torch.float32, device=self.device)
                self._opt_hyper_host = torch.zeros(8, dtype=torch.float32, pin_memory=True)
            K.adamw_hyper(self._opt_hyper_host, lr=lr, beta1=beta1, beta2=beta2, step=step, eps=eps, weight_decay=weight_decay, seed=seed_base)
            self._opt_hyper.copy_(self._opt_hyper_host, non_blocking=True)

            def adam_all():
                for idx, (name, master, spec, l) in enumerate(items):
                    am = w._stat(l, spec.name)[0:1] if (l is not None and spec.name in MATRICES and w.quantized) else None
                    if master.numel() % 8:
                        raise ValueError(f"parameter shard {name} has {master.numel()} elements; shard sizes must be multiples of 8")
                    K.adamw(master.view(-1), shard_of[name].view(-1), o.m[name].view(-1), o.v[name].view(-1), lr=0.0, beta1=0.0, beta2=0.0,
                            step=1, eps=0.0, weight_decay=1.0 if spec.matrix else 0.0, grad_scale=scale, absmax=am,
                            m_scales=o.m_scales.get(name), seed=idx * 7919, elem_offset=self.comm.rank * master.numel(), hyper=self._opt_hyper)
            self.graphs.run(("opt-adamw",), adam_all)
            items = []                                           # the staged loop below has nothing left to do
        stager = self._stager
        staged = [None] * len(items)

        def prefetch(i):
            name, master, spec, l = items[i]
            par = i & 1
            staged[i] = (stager.fetch(master, "p", par), stager.fetch(shard_of[name], "g", par),
                         stager.fetch(o.m[name], "m", par), stager.fetch(o.v[name], "v", par))

        if items:
            prefetch(0)
        main = torch.cuda.current_stream(self.device) if self.device.type == "cuda" else None
        for idx, (name, master, spec, l) in enumerate(items):
            if idx + 1 < len(items):
                prefetch(idx + 1)                      # H2D of the next tensor's state overlaps this tensor's update
            (pm, e0), (gm, e1), (mm, e2), (vm, e3) = staged[idx]
            staged[idx] = None
            for e in (e0, e1, e2, e3):
                if e is not None:
                    main.wait_event(e)
            ms = o.m_scales.get(name)
            wd = weight_decay if spec.matrix else 0.0
            am = w._stat(l, spec.name)[0:1] if (l is not None and spec.name in MATRICES and w.quantized) else None
            n = pm.numel()
            if n % 8:
                raise ValueError(f"parameter shard {name} has {n} elements; shard sizes must be multiples of 8")
            K.adamw(pm.view(-1), gm.view(-1), mm.view(-1), vm.view(-1), lr=lr, beta1=beta1, beta2=beta2, step=step, eps=eps,
                    weight_decay=wd, grad_scale=scale, absmax=am, m_scales=ms, seed=seed_base + idx * 7919,
                    elem_offset=self.comm.rank * master.numel())
            par = idx & 1
            stager.mark_consumed(par)
            stager.store(pm, master, "p", par)
            stager.store(mm, o.m[name], "m", par)
            stager.store(vm, o.v[name], "v", par)
        stager.finish()
        w.sync_absmax(recompute=False)
        w.invalidate()
        g.end_step()
        self.rng_state = (self.rng_state * 48271) % 2147483647
        loss, loss1k = self._reduce_loss(self.B * self.T * grad_accum)
        ntok = float(self.B * self.T * grad_accum)
        hs = self.host_scalars
        hs[0:2].copy_(self.norm_io, non_blocking=True)
        hs[2:4].copy_(self.lse_stats, non_blocking=True)
        self._mark("optimizer")
        if self.device.type == "cuda":
            torch.cuda.current_stream().synchronize()
        nvtx.pop(r_upd)
        res = {"loss": loss, "loss_1k": loss1k, "norm": float(hs[0]), "z_max": float(hs[2]), "z_mean": float(hs[3]) / ntok}
        if self.opts.trigger_timing_events:
            res["time_breakdown"] = self.time_breakdown()
        return res

    # ================================================================================== introspection
    def get_gradients(self) -> Dict[str, torch.Tensor]:
        """Local gradient shards by checkpoint name (for tests and the Python API)."""
        out = {}
        for name, master, spec, l in self.weights.master_items():
            out[name] = self.grads.get_block_shard(l)[spec.name] if l is not None else self.grads.get_nb_shard(spec.name)
        return out
