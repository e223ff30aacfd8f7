"""``pyllmq-train``: a training run written against the Python API only.

Where ``python -m llmq_b200.cli.train`` is the counterpart of the reference's ``train`` executable (one rank per
process, every rank runs the loop), this script is the counterpart of the reference's second front end,
scripts/train.py:16-273: ONE Python process owns the loop and drives all GPUs through ``LLMQTrainer`` (which starts one
worker per GPU), feeds them from a single ``DataLoader`` with ``gpus * batch`` rows per micro-step, and writes the run
log through ``training_logger_context``.  Evaluation / checkpoint cadence, checkpoint retention, resume, learning-rate
schedule and the final export all go through public API calls, so the script doubles as a usage example.

    python -m llmq_b200.scripts.train --model Qwen2.5-0.5B --from-scratch --train-file "data/train-*.bin" \
        --eval-file "data/eval-*.bin" --batch-size 8 --seq-length 1024 --grad-accumulation 8 --matmul-dtype e4m3 --gpus 2
"""
from __future__ import annotations

import argparse
import glob
import os
import sys
import time
from typing import Optional, Tuple

import numpy as np

import pyllmq


def setup_options(config: pyllmq.TrainingConfig) -> pyllmq.LLamaOptions:
    """``LLamaOptions`` from the parsed flags.  ``TrainingConfig.to_options`` applies the flag relations of the
    command line (recompute-block implies att + ffn + norm, zero levels imply the shard flags, ...)."""
    return config.to_options()


def _token_buffers(config: pyllmq.TrainingConfig) -> Tuple[np.ndarray, np.ndarray]:
    rows = max(1, config.gpus) * config.batch_size
    return np.empty((rows, config.seq_len), dtype=np.int32), np.empty((rows, config.seq_len), dtype=np.int32)


def run_evaluation(trainer: pyllmq.LLMQTrainer, eval_loader: Optional[pyllmq.DataLoader], in_tokens: np.ndarray, out_tokens: np.ndarray,
                   max_steps: int) -> Tuple[float, float, int, int]:
    """(mean loss, mean loss over the first 1024 positions, milliseconds, batches) over at most ``max_steps`` batches from
    the start of the validation set."""
    if eval_loader is None:
        return 0.0, 0.0, 0, 0
    t0 = time.time()
    eval_loader.set_state(eval_loader.seed, 0, 0, 0)
    rows = in_tokens.shape[0]
    total, total_1k, batches = 0.0, 0.0, 0
    while batches < max_steps and eval_loader.has_next(rows):
        eval_loader.load_batch(in_tokens, out_tokens)
        loss, loss_1k = trainer.validate(in_tokens, out_tokens)
        total, total_1k, batches = total + loss, total_1k + loss_1k, batches + 1
    if batches == 0:
        print("WARNING: insufficient validation data", file=sys.stderr)
        return 0.0, 0.0, 0, 0
    return total / batches, total_1k / batches, int((time.time() - t0) * 1000), batches


def parse_args(argv=None) -> pyllmq.TrainingConfig:
    parser = argparse.ArgumentParser(description="Train a Llama / Qwen2 decoder through the Python API")
    pyllmq.add_training_args(parser)
    ns = parser.parse_args(argv)
    fields = set(pyllmq.TrainingConfig.__dataclass_fields__)
    config = pyllmq.TrainingConfig(**{k: v for k, v in vars(ns).items() if k in fields}).finalize()
    if config.gpus <= 0:
        config.gpus = max(1, pyllmq.get_num_gpus())
    return config


def create_trainer(config: pyllmq.TrainingConfig, options: pyllmq.LLamaOptions) -> Tuple[pyllmq.LLMQTrainer, int, dict]:
    """The trainer in one of its three starting states: resumed from a checkpoint, random init, or imported weights.
    Returns (trainer, first step, checkpoint meta data)."""
    kw = dict(ngpu=config.gpus, options=options, batch_size=config.batch_size, seq_len=config.seq_len, grad_accum=config.grad_accumulation,
              memcpy_all_gather=config.memcpy_all_gather, memcpy_send_recv=config.memcpy_send_recv)
    if config.continue_from_checkpoint is not None:
        c = config.continue_from_checkpoint                        # "latest" (bare --continue), a step number, or a directory
        root = config.checkpoint_dir if (c in ("", "latest") or c.isdigit()) else c
        step = int(c) if c.isdigit() else pyllmq.find_latest_checkpoint(root)
        if step < 0:
            raise FileNotFoundError(f"no checkpoint found in {root}")
        model_cfg = pyllmq.Config.from_name(config.model, config.model_dtype) if config.from_scratch \
            else pyllmq.Config.from_pretrained(config.model, config.model_dtype)
        trainer = pyllmq.LLMQTrainer(config=model_cfg, **kw)
        print(f"Loading checkpoint from step {step}...")
        meta = trainer.load_checkpoint(root, step)
        return trainer, int(meta["run"]["step"]), meta
    if config.from_scratch:
        print(f"Creating {config.model} from scratch...")
        trainer = pyllmq.LLMQTrainer(config=pyllmq.Config.from_name(config.model, config.model_dtype), **kw)
        trainer.init_weights()
        return trainer, 0, {}
    print(f"Loading model from {config.model}...")
    trainer = pyllmq.LLMQTrainer.from_pretrained(name=config.model, dtype=config.model_dtype, **kw)
    return trainer, 0, {}


def run_training_loop(config: pyllmq.TrainingConfig, trainer: pyllmq.LLMQTrainer, eval_loader: Optional[pyllmq.DataLoader],
                      train_loader: pyllmq.DataLoader, first_step: int, logger: pyllmq.TrainingRunLogger, lr_schedule) -> dict:
    in_tokens, out_tokens = _token_buffers(config)
    rows = in_tokens.shape[0]
    step_tokens = rows * config.seq_len * config.grad_accumulation
    result: dict = {}
    for step in range(first_step, config.steps):
        if config.ckpt_interval > 0 and step % config.ckpt_interval == 0 and step > first_step and config.save_training_state:
            trainer.save_checkpoint(config.checkpoint_dir, step, {"data-loader": train_loader.get_state()})
            if config.ckpt_keep_n > 0:
                removed = pyllmq.clean_old_checkpoints(config.checkpoint_dir, config.ckpt_keep_n, config.ckpt_major)
                if removed:
                    logger.log_message(step, f"cleaned {len(removed)} checkpoints")
        if config.eval_every > 0 and step % config.eval_every == 0 and step > first_step:
            loss, loss_1k, ms, batches = run_evaluation(trainer, eval_loader, in_tokens, out_tokens, config.eval_num_steps)
            if batches:
                logger.log_eval(step, batches * rows * config.seq_len, ms, loss, loss_1k)
        t0 = time.time()
        for _ in range(config.grad_accumulation):
            if not train_loader.has_next(rows):
                train_loader.advance_epoch()
            train_loader.load_batch(in_tokens, out_tokens)
            trainer.step(in_tokens, out_tokens, config.z_loss)      # returns once queued: the next batch loads meanwhile
        if config.log_gpu_util > 0 and step % config.log_gpu_util == 0:
            for gpu_id, info in enumerate(trainer.get_gpu_info()):
                logger.log_gpu_state(step, gpu_id, info)
        lr = lr_schedule.get_lr(step)
        result = trainer.update(lr, config.beta_1, config.beta_2, step + 1, config.weight_decay, config.grad_clip, config.adam_epsilon)
        logger.log_step(step, step_tokens, (time.time() - t0) * 1e3, result["norm"], result["loss"], result["loss_1k"], result["z_max"],
                        result["z_mean"], lr)
    return result


def main(argv=None) -> int:
    config = parse_args(argv)
    options = setup_options(config)
    os.makedirs(config.checkpoint_dir, exist_ok=True)
    os.makedirs(config.out_dir, exist_ok=True)
    with pyllmq.training_logger_context(config) as logger:
        logger.log_cmd(argv if argv is not None else sys.argv)
        train_files = sorted(glob.glob(config.train_file))
        eval_files = sorted(glob.glob(config.eval_file))
        if not train_files:
            raise FileNotFoundError(f"no training token files match {config.train_file}")
        train_loader = pyllmq.DataLoader(train_files, config.seq_len, seed=config.train_seed)
        eval_loader = pyllmq.DataLoader(eval_files, config.seq_len, seed=config.eval_seed) if eval_files else None
        logger.log_dataset(train_loader, eval_loader)

        trainer, first_step, meta = create_trainer(config, options)
        model_vocab = trainer.config.vocab_size
        for what, loader in (("training", train_loader), ("validation", eval_loader)):
            if loader is not None and loader.vocab_size > model_vocab:
                raise ValueError(f"model vocab size {model_vocab} does not match {what} data vocab size {loader.vocab_size}")
        state = meta.get("data-loader") if meta else None
        if state and not config.new_data:
            train_loader.set_state(state["seed"], state["epoch"], state["file_index"], state["chunk_index"])

        rows = max(1, config.gpus) * config.batch_size
        step_tokens = rows * config.seq_len * config.grad_accumulation
        steps_per_epoch = max(1, train_loader.num_tokens // step_tokens)
        if config.steps <= 0:
            config.steps = steps_per_epoch * max(1, config.epochs)
        lr_schedule = pyllmq.CosineLRSchedule(config.learning_rate, config.steps, config.warmup_steps,
                                              config.learning_rate * config.final_lr_fraction)
        for gpu_id in range(config.gpus):
            logger.log_allocator(trainer, gpu_id)
        logger.set_expected_time_per_token(trainer)           # speed-of-light estimate for the SOL % column
        print(f"Starting at step {first_step}: {config.steps} steps of {step_tokens} tokens, {steps_per_epoch} steps per epoch")

        run_training_loop(config, trainer, eval_loader, train_loader, first_step, logger, lr_schedule)

        in_tokens, out_tokens = _token_buffers(config)
        loss, loss_1k, ms, batches = run_evaluation(trainer, eval_loader, in_tokens, out_tokens, 1 << 30)
        if batches:
            logger.log_eval(config.steps, batches * rows * config.seq_len, ms, loss, loss_1k)
            print(f"Final validation loss: {loss:.4f}")
        if config.save_training_state:
            trainer.save_checkpoint(config.checkpoint_dir, config.steps, {"data-loader": train_loader.get_state()})
        print(f"Saving model to {config.out_dir}...")
        trainer.export_model(config.out_dir)
        trainer.close()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
