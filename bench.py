#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s, whole job) of Qwen2.5-7B-arch with e4m3 matmuls.

    python bench.py --gpus N --steps K --warmup W            (N == 1)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \
        bench.py --gpus N --steps K --warmup W               (N > 1, one rank per GPU)

Config (weak scaling, fixed per-GPU work): per-GPU batch 8 x seq 2048 uniform-random tokens, random-init bf16
master weights, e4m3 matmuls, bf16 AdamW moments, recompute-swiglu; with N > 1 weights, gradients and optimizer
state are sharded (all-gather before each layer).  A step is forward + backward + clip + AdamW.

Two measurements are reported in one JSON line:
* ``value``  - device time (CUDA events) of K steps fed from device-resident token tensors, max over ranks;
* ``e2e``    - the same K steps through the public API (``LLMQTrainer.step`` / ``update``) with, every step, the
  host->device copy of that step's tokens from pinned memory and the device->host read of loss and norm.
Every step streams far more than the 126 MB L2 (weights + activations are tens of GB), so no explicit flush is needed.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

BASELINE_TOKS_PER_GPU = None       # the reference publishes no B200 number


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through nvidia-smi while the timed region runs."""

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag = index, [], threading.Event()

    def run(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        while not self.stop_flag.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={q}", "--format=csv,noheader,nounits", "-i", str(self.index)],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            self.stop_flag.wait(0.2)

    def summary(self):
        sm = sorted(int(float(s[0])) for s in self.samples if s and s[0].replace(".", "").isdigit())
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            for n, v in zip(names, s[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mx = max((int(float(s[1])) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()), default=None)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(sm)}


def reference_arm(args):
    """Runs the UNMODIFIED reference: ``baseline/_ref/ref_bench`` is ``baseline/ref_harness.cpp`` linked against the
    reference's own ``llmq-common`` library, built offline from the reference sources by ``baseline/build_ref.py``.
    The reference drives all N GPUs from one process (one rank thread per GPU, train.cpp:269-291), so under
    ``torch.distributed.run`` only local rank 0 starts it and the other ranks leave quietly.  Nothing of this
    repository's package or kernel libraries is imported on this path."""
    if int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0"))) != 0:
        return 0
    exe = os.path.join(ROOT, "baseline", "_ref", "ref_bench")
    if not os.path.exists(exe):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/ref_bench is not built (python baseline/build_ref.py needs the reference sources)"}))
        return 0
    GA = args.grad_accum
    cmd = [exe, "--model", args.model, "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup),
           "--batch", str(args.batch), "--seq-len", str(args.seq_len), "--grad-accumulation", str(GA),
           "--matmul-dtype", args.matmul_dtype, "--lmhead-chunks", str(args.lmhead_chunks), "--use-cuda-graphs"]
    zl = args.zero_level or (1 if args.gpus == 1 else 3)
    cmd += ["--zero-level", str(zl)]
    if args.recompute == "swiglu":
        cmd.append("--recompute-swiglu")
    elif args.recompute == "block":
        cmd.append("--recompute-block")
    if args.offload_master:
        cmd.append("--offload-master")
    if args.offload_opt:
        cmd += ["--offload-opt-m", "--offload-opt-v"]
    if args.persistent_quants:
        cmd.append("--persistent-quants")
    env = dict(os.environ)
    for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE", "MASTER_ADDR", "MASTER_PORT"):     # the reference's threads mode needs none of these
        env.pop(k, None)
    sampler = ClockSampler(0)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
    result = None
    for line in proc.stdout:
        line = line.strip()
        if line == "TIMED_BEGIN":
            sampler.start()
        elif line == "TIMED_END":
            sampler.stop_flag.set()
        elif line.startswith("{"):
            result = json.loads(line)
    err = proc.stderr.read()
    rc = proc.wait()
    sampler.stop_flag.set()
    if rc != 0 or result is None or "unavailable" in result:
        why = (result or {}).get("unavailable") or f"reference harness exited {rc}: {err.strip().splitlines()[-1] if err.strip() else 'no output'}"
        print(json.dumps({"impl": "reference", "unavailable": why[:300]}))
        sys.stderr.write(err[-4000:])
        return 0
    B, T, N = args.batch, args.seq_len, args.gpus
    value = result["device_tok_s"]
    out = {
        "metric": f"train tokens/sec/box {args.model} {args.matmul_dtype}", "value": value, "unit": "tokens/s", "n_gpus": N,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": result["device_ms"] / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": f"bf16 model / {args.matmul_dtype} matmul",
        "data": "synthetic uniform-random tokens, random-init weights",
        "config": {"model": args.model, "global_batch": B * N * GA, "seq_len": T, "per_gpu_batch": B, "grad_accum": GA,
                   "parallelism": f"dp{N}" + ("" if N == 1 else f"-zero{zl}"), "recompute": args.recompute, "opt_moments": "bf16",
                   "lmhead_chunks": args.lmhead_chunks, "cuda_graphs": True, "launch": "one process, one rank thread per GPU (the reference's threads mode)",
                   "offload": [n for n, on in (("master", args.offload_master), ("adam_m", args.offload_opt), ("adam_v", args.offload_opt)) if on],
                   "persistent_quants": args.persistent_quants,
                   "l2": "every step streams >60 GB of weights+activations (>> 126 MB L2), no flush needed"},
        "clocks": sampler.summary() if sampler.samples else {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0},
        "e2e": {"value": result["e2e_tok_s"], "unit": "tokens/s", "ms_per_step": result["e2e_ms"] / args.steps,
                "h2d_bytes_per_step": result["h2d_bytes_per_step"], "d2h_bytes_per_step": result["d2h_bytes_per_step"],
                "timing": "host wall clock around K steps incl. filling the pinned token buffers, the H2D copies in forward() and the host reads of loss and norm"},
        "gpu_launches": None, "loss": result["loss"], "impl": "reference",
        "build": "unmodified reference sources compiled offline for sm_100a (baseline/build_ref.py): cuBLASLt + cuDNN + NCCL",
    }
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="Qwen2.5-7B")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--grad-accum", type=int, default=1)
    ap.add_argument("--matmul-dtype", default="e4m3")
    ap.add_argument("--lmhead-chunks", type=int, default=4)
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (the result is then not the headline metric)")
    ap.add_argument("--collectives", default="auto")
    ap.add_argument("--recompute", default="swiglu", choices=["none", "swiglu", "block"], help="headline config: swiglu")
    ap.add_argument("--offload-master", action="store_true")
    ap.add_argument("--offload-opt", action="store_true", help="Adam moments in pinned host memory (the 14B configuration)")
    ap.add_argument("--persistent-quants", action="store_true",
                    help="ZeRO-3: keep the quantised weight shards on the device for the whole optimizer step (master weights are read once)")
    ap.add_argument("--fuse-swiglu", type=int, default=None)
    ap.add_argument("--overlap-dw", type=int, default=None)
    ap.add_argument("--overlap-lmhead", type=int, default=None)
    ap.add_argument("--lmhead-transpose-dlogits", type=int, default=None)
    ap.add_argument("--swiglu-two-pass", type=int, default=None, help="0 = SwiGLU backward writes bf16 then quantises, 1 = abs-max pass + quantising pass (default)")
    ap.add_argument("--kmajor-backward", type=int, default=None, help="0 = backward GEMMs read MN-major operands in place, 1 = transposed fp8 copies (default)")
    ap.add_argument("--cuda-graphs", type=int, default=-1,
                    help="1 = replay per-block CUDA graphs (the reference's --use-cuda-graphs; default), 0 = plain launches")
    ap.add_argument("--gather-behind-first-gemm", type=int, default=None, help="ZeRO-3: 1 = weight gathers start beside attention, 0 = at the top of the previous block (default)")
    ap.add_argument("--time-breakdown", action="store_true", help="diagnostic: print milliseconds per phase of the last timed step to stderr (adds a synchronisation per step)")
    ap.add_argument("--memcpy-all-gather", action="store_true", help="weight all-gathers as copy-engine transfers instead of SM stores")
    ap.add_argument("--memcpy-send-recv", action="store_true", help="with --all-to-all-reduce: gradient exchange as copy-engine transfers")
    ap.add_argument("--all-to-all-reduce", action="store_true")
    ap.add_argument("--zero-level", type=int, default=0, help="0 = pick from --gpus (1 GPU: unsharded, else 3)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)

    from llmq_b200 import api
    from llmq_b200.config import create_config_from_name
    from llmq_b200.ops import lib as L
    from llmq_b200.options import LLamaOptions

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            print(f"bench.py --gpus {args.gpus} must be started with torch.distributed.run (one rank per GPU)", file=sys.stderr)
            return 2
    cfg = create_config_from_name(args.model, "bf16")
    if args.layers:
        cfg = cfg.replace(num_hidden_layers=args.layers)
    opts = LLamaOptions(recompute_swiglu=args.recompute == "swiglu", recompute_block=args.recompute == "block",
                        offload_master=args.offload_master, matmul_type=args.matmul_dtype, momentum_type="bf16", variance_type="bf16",
                        lmhead_chunks=args.lmhead_chunks, collectives=args.collectives, use_cuda_graphs=(args.cuda_graphs != 0))
    if args.fuse_swiglu is not None:
        opts.fuse_swiglu = args.fuse_swiglu
    if args.overlap_dw is not None:
        opts.overlap_dw = bool(args.overlap_dw)
    if args.overlap_lmhead is not None:
        opts.overlap_lmhead = bool(args.overlap_lmhead)
    if args.lmhead_transpose_dlogits is not None:
        opts.lmhead_transpose_dlogits = bool(args.lmhead_transpose_dlogits)
    if args.kmajor_backward is not None:
        opts.kmajor_backward = bool(args.kmajor_backward)
    if args.swiglu_two_pass is not None:
        opts.swiglu_backward_two_pass = bool(args.swiglu_two_pass)
    zl = args.zero_level or (1 if args.gpus == 1 else 3)
    opts.set_zero_level(zl)
    opts.offload_opt_m = opts.offload_opt_v = args.offload_opt
    opts.persistent_quants = args.persistent_quants
    B, T, GA = args.batch, args.seq_len, args.grad_accum
    opts.use_all_to_all_reduce = bool(args.all_to_all_reduce)
    opts.trigger_timing_events = bool(args.time_breakdown)
    if args.gather_behind_first_gemm is not None:
        opts.gather_behind_first_gemm = bool(args.gather_behind_first_gemm)
    trainer = api.LLMQTrainer(ngpu=args.gpus, config=cfg, options=opts, batch_size=B, seq_len=T, grad_accum=GA,
                              memcpy_all_gather=args.memcpy_all_gather, memcpy_send_recv=args.memcpy_send_recv)
    trainer.init_weights()
    dev, comm, rank = trainer.device, trainer.comm, trainer.rank
    gen = torch.Generator().manual_seed(1234 + rank)
    n_batches = min(256, GA * (args.warmup + 2 * args.steps))      # fresh tokens every micro-step (cycled only beyond 256)
    host_tokens = [torch.randint(0, cfg.vocab_size, (B, T + 1), generator=gen, dtype=torch.int32) for _ in range(n_batches)]
    host_in = [t[:, :-1].contiguous().pin_memory() for t in host_tokens]
    host_tg = [t[:, 1:].contiguous().pin_memory() for t in host_tokens]
    dev_in = [t.to(dev) for t in host_in]
    dev_tg = [t.to(dev) for t in host_tg]
    lr = 1e-5

    def run_step(i, step_no, from_host):
        for j in range(GA):
            k = ((step_no - 1) * GA + j) % n_batches
            if from_host:
                trainer.step(host_in[k], host_tg[k])
            else:
                trainer.step(dev_in[k], dev_tg[k])
        return trainer.update(lr, 0.9, 0.95, step_no, 0.1, 1.0)

    def sync_all():
        comm.barrier()
        torch.cuda.synchronize()

    step_no = 0
    for i in range(args.warmup):
        step_no += 1
        res = run_step(i, step_no, False)
    sync_all()
    sampler = ClockSampler(dev.index or 0)
    sampler.start()
    l0 = L.launch_count
    loss_host = None

    def device_region():
        nonlocal step_no, res
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        sync_all()
        e0.record()
        for i in range(args.steps):
            step_no += 1
            res = run_step(i, step_no, False)
        e1.record()
        sync_all()
        return e0.elapsed_time(e1)

    def e2e_region():
        # end to end through the public API: pinned-host inputs every step, the step's loss and norm read on the host
        nonlocal step_no, res, loss_host
        sync_all()
        t0 = time.perf_counter()
        for i in range(args.steps):
            step_no += 1
            res = run_step(i, step_no, True)
            loss_host = res["loss"]
        sync_all()
        return (time.perf_counter() - t0) * 1e3

    if os.environ.get("LLMQ_BENCH_E2E_FIRST", "0") == "1":      # diagnostic: which of the two regions runs first
        ms_e2e = e2e_region()
        l0 = L.launch_count
        ms_dev = device_region()
        launches = L.launch_count - l0
    else:
        ms_dev = device_region()
        launches = L.launch_count - l0
        if args.time_breakdown and isinstance(res, dict) and res.get("time_breakdown"):
            print(f"[rank {rank}] phases of the last step (ms): " + ", ".join(f"{k} {v:.1f}" for k, v in res["time_breakdown"].items()), file=sys.stderr)
        ms_e2e = e2e_region()
    sampler.stop_flag.set()
    sampler.join(timeout=3)
    t = torch.tensor([ms_dev, ms_e2e], dtype=torch.float64, device=dev)
    if comm.world > 1:
        comm.all_reduce(t, "max").wait()
    ms_dev, ms_e2e = float(t[0]), float(t[1])
    from llmq_b200.ops import kernels as K
    K.check_status(dev)
    tokens = B * T * GA * comm.world * args.steps
    value = tokens / (ms_dev / 1e3)
    e2e = tokens / (ms_e2e / 1e3)
    if rank == 0:
        # SOL % as the reference defines it (spec-sheet peaks: bf16 2200 / fp8 4500 TFLOP/s for B200)
        from llmq_b200.utils.sol import estimate_speed_of_light
        sol_ns = estimate_speed_of_light(cfg, T, torch.bfloat16, opts.matmul_dtype(), comm.world)
        sol_pct = 100.0 * sol_ns / (1e9 / value) if sol_ns > 0 else None
        out = {
            "metric": f"train tokens/sec/box {args.model} {args.matmul_dtype}", "value": value, "unit": "tokens/s", "n_gpus": comm.world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_dev / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": (value / (BASELINE_TOKS_PER_GPU * comm.world)) if BASELINE_TOKS_PER_GPU else None,
            "dtype": f"bf16 model / {args.matmul_dtype} matmul", "data": "synthetic uniform-random tokens, random-init weights",
            "config": {"model": args.model + ("" if not args.layers else f"[layers={args.layers}]"), "global_batch": B * comm.world * GA,
                       "seq_len": T, "per_gpu_batch": B, "grad_accum": GA,
                       "parallelism": f"dp{comm.world}" + ("" if comm.world == 1 else f"-zero{zl}"), "recompute": args.recompute,
                       "opt_moments": "bf16", "lmhead_chunks": args.lmhead_chunks,
                       "offload": [n for n, on in (("master", args.offload_master), ("adam_m", args.offload_opt), ("adam_v", args.offload_opt)) if on],
                       "persistent_quants": args.persistent_quants,
                       "l2": "every step streams >60 GB of weights+activations (>> 126 MB L2), no flush needed"},
            "clocks": sampler.summary(),
            "e2e": {"value": e2e, "unit": "tokens/s", "ms_per_step": ms_e2e / args.steps, "h2d_bytes_per_step": 2 * B * T * 4 * GA,
                    "d2h_bytes_per_step": 32, "timing": "host wall clock around K steps incl. pinned H2D token copies and D2H loss/norm"},
            "gpu_launches": launches, "loss": loss_host, "sol_pct_of_spec_sheet_peak": sol_pct, "impl": "ours",
        }
        print(json.dumps(out))
    trainer.close()
    trainer.comm.shutdown()
    return 0


if __name__ == "__main__":
    sys.exit(main())
