"""``pyllmq-demo``: minimal use of the Python API - a small model trained from scratch on synthetic tokens."""
from __future__ import annotations

import argparse
import time

import numpy as np

import llmq_b200.api as api
from llmq_b200.options import LLamaOptions


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("--model", default="Qwen2.5-0.5B")
    p.add_argument("--steps", type=int, default=10)
    p.add_argument("--batch", type=int, default=4)
    p.add_argument("--seq-len", type=int, default=1024)
    p.add_argument("--matmul-dtype", default="e4m3")
    a = p.parse_args(argv)
    cfg = api.Config.from_name(a.model, "bf16")
    opts = LLamaOptions(matmul_type=a.matmul_dtype, recompute_swiglu=True, momentum_type="bf16", variance_type="bf16")
    tr = api.LLMQTrainer(ngpu=1, config=cfg, options=opts, batch_size=a.batch, seq_len=a.seq_len, grad_accum=1)
    tr.init_weights()
    rng = np.random.default_rng(0)
    data = rng.integers(0, cfg.vocab_size, size=(a.batch, a.seq_len + 1), dtype=np.int32)   # one batch, memorised
    for step in range(a.steps):
        t0 = time.time()
        tr.step(np.ascontiguousarray(data[:, :-1]), np.ascontiguousarray(data[:, 1:]))
        r = tr.update(3e-4, 0.9, 0.95, step + 1, 0.1, 1.0)
        print(f"step {step:3d} loss {r['loss']:.4f} norm {r['norm']:.3f} {a.batch * a.seq_len / (time.time() - t0):.0f} tok/s")
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
