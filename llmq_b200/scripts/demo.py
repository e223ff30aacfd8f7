"""``pyllmq-demo``: a tour of the Python API in one file (role of the reference's scripts/demo.py).

It spells out a model architecture by hand, picks training options, writes a small synthetic token file pair when no data
is given, trains from a random initialisation with gradient accumulation while the next batch loads, prints the memory
report and (on GPUs) the telemetry the trainer exposes, validates, saves a checkpoint, restores it into a second trainer to
show that the state round-trips, and exports a Hugging Face compatible model directory.

    python -m llmq_b200.scripts.demo                      # tiny model, runs on CPU or GPU in seconds
    python -m llmq_b200.scripts.demo --preset Qwen2.5-0.5B --matmul-dtype e4m3 --batch 2 --seq-len 1024 --steps 100
"""
from __future__ import annotations

import argparse
import os
import tempfile
import time

import numpy as np

import pyllmq
from llmq_b200.training.dataloader import write_synthetic_token_file


def build_config(preset: str) -> "pyllmq.Config":
    if preset:
        return pyllmq.Config.from_name(preset, "bf16")
    # every field of the architecture can be given explicitly; this is a 4-layer Qwen2-style decoder
    return pyllmq.Config(architecture="qwen2", hidden_size=256, intermediate_size=768, max_position_embeddings=4096,
                         num_attention_heads=4, num_hidden_layers=4, num_key_value_heads=2, rms_norm_eps=1e-6,
                         tie_word_embeddings=True, dtype="bfloat16", vocab_size=4096)


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    p.add_argument("--preset", default="", help="a built-in architecture name (e.g. Qwen2.5-0.5B) instead of the hand-written small model")
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--eval-steps", type=int, default=4)
    p.add_argument("--batch", type=int, default=2)
    p.add_argument("--seq-len", type=int, default=256)
    p.add_argument("--grad-accumulation", type=int, default=2)
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--matmul-dtype", default="", help="e4m3 for fp8 matmuls on a GPU; empty = the model dtype")
    p.add_argument("--model-dtype", default="", help="default: bf16 on a GPU, fp32 on the CPU")
    p.add_argument("--data-dir", default="", help="directory with train-*.bin / eval-*.bin token files; default: synthetic tokens")
    p.add_argument("--out-dir", default="demo-model")
    a = p.parse_args(argv)

    on_gpu = pyllmq.get_num_gpus() > 0
    config = build_config(a.preset)
    dtype = a.model_dtype or ("bf16" if on_gpu else "fp32")
    from llmq_b200.config import parse_dtype
    config = config.replace(dtype=parse_dtype(dtype))

    # recompute the activation in backward instead of storing it; never materialise the full logit tensor; Adam moments in bf16
    opt_dtype = "bf16" if dtype == "bf16" else "fp32"
    options = pyllmq.LLamaOptions(recompute_swiglu=True, lmhead_chunks=2, momentum_type=opt_dtype, variance_type=opt_dtype,
                                  matmul_type=a.matmul_dtype or None)

    lr, beta_1, beta_2, weight_decay, grad_clip = 3e-4, 0.9, 0.95, 1e-2, 1.0
    rows = a.gpus * a.batch

    work = tempfile.mkdtemp(prefix="pyllmq-demo-")
    data_dir = a.data_dir
    if not data_dir:
        print("generating synthetic token files...")
        data_dir = work
        n_train = rows * (a.seq_len + 1) * a.grad_accumulation * (a.steps + 2)
        write_synthetic_token_file(os.path.join(work, "train-000.bin"), max(n_train, 50_000), config.vocab_size, seed=0)
        write_synthetic_token_file(os.path.join(work, "eval-000.bin"), rows * (a.seq_len + 1) * (a.eval_steps + 2), config.vocab_size, seed=1)
    # it is not required to use pyllmq.DataLoader: any int32 arrays of shape (gpus * batch, seq_len) will do
    in_tokens = np.empty((rows, a.seq_len), dtype=np.int32)
    out_tokens = np.empty((rows, a.seq_len), dtype=np.int32)
    train_loader = pyllmq.DataLoader(os.path.join(data_dir, "train-*.bin"), a.seq_len, 42)
    eval_loader = pyllmq.DataLoader(os.path.join(data_dir, "eval-*.bin"), a.seq_len, 42)

    print("creating trainer...")
    trainer = pyllmq.LLMQTrainer(ngpu=a.gpus, config=config, options=options, batch_size=a.batch, seq_len=a.seq_len,
                                 grad_accum=a.grad_accumulation)
    print("initializing weights...")
    trainer.init_weights()
    # alternative: pyllmq.LLMQTrainer.from_pretrained("Qwen/Qwen2.5-0.5B", ngpu=1, dtype="bf16", options=options, ...)

    print("\nmemory consumption:")
    for name, where in trainer.get_allocator_info(0).items():
        print(f" {name:20}: {where.get('device', 0) // 1024 // 1024:6} MiB device {where.get('pinned', 0) // 1024 // 1024:6} MiB pinned")

    print("\nstarting training...\n")
    train_loader.load_batch(in_tokens, out_tokens)
    first_loss = last_loss = None
    t0 = time.perf_counter()
    for step in range(a.steps):
        for _ in range(a.grad_accumulation):
            trainer.step(in_tokens, out_tokens)              # queued asynchronously ...
            if not train_loader.has_next(rows):
                train_loader.advance_epoch()
            train_loader.load_batch(in_tokens, out_tokens)   # ... so the next batch loads while the GPU works
        if on_gpu and step % 10 == 0:
            for info in trainer.get_gpu_info():
                print(f"             power: {info.power // 1000:4}W  temp: {info.temperature:3}C  clock: {info.clock / 1000:3.1f}GHz  "
                      f"throttle: {info.throttle_reason}")
        result = trainer.update(lr, beta_1, beta_2, step + 1, weight_decay, grad_clip)
        now = time.perf_counter()
        print(f"step: {step:5}  loss: {result['loss']:6.3f}  norm: {result['norm']:6.3f}  time: {now - t0:6.3f}s")
        t0 = now
        first_loss = result["loss"] if first_loss is None else first_loss
        last_loss = result["loss"]

    print("\neval...")
    val, n = 0.0, 0
    while n < a.eval_steps and eval_loader.has_next(rows):
        eval_loader.load_batch(in_tokens, out_tokens)
        val += trainer.validate(in_tokens, out_tokens)[0]
        n += 1
    print(f"eval loss: {val / max(n, 1):6.3f}")

    # checkpoints hold master weights, optimizer state and the step; a fresh trainer continues exactly where this one stopped
    ckpt_dir = os.path.join(work, "ckpt")
    trainer.save_checkpoint(ckpt_dir, a.steps)
    again = pyllmq.LLMQTrainer(ngpu=a.gpus, config=config, options=options, batch_size=a.batch, seq_len=a.seq_len,
                               grad_accum=a.grad_accumulation)
    again.load_checkpoint(ckpt_dir, pyllmq.find_latest_checkpoint(ckpt_dir))
    eval_loader.set_state(eval_loader.seed, 0, 0, 0)
    eval_loader.load_batch(in_tokens, out_tokens)
    a_loss, b_loss = trainer.validate(in_tokens, out_tokens)[0], again.validate(in_tokens, out_tokens)[0]
    print(f"restored trainer reproduces the validation loss: {a_loss:.6f} vs {b_loss:.6f}")
    again.close()

    trainer.export_model(a.out_dir)
    print(f"exported a Hugging Face compatible model to {a.out_dir} (first loss {first_loss:.3f}, last loss {last_loss:.3f})")
    trainer.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
