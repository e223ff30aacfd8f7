"""``train``: pre-training / full fine-tuning driver with the flags of the reference CLI (train.cpp).

    python -m llmq_b200.cli.train --model Qwen2.5-0.5B --from-scratch --matmul-dtype e4m3 --gpus 8 ...

Ranks: with a launcher environment (torchrun's RANK/WORLD_SIZE or Open MPI's OMPI_COMM_WORLD_*) this process is
one rank.  Otherwise ``--gpus N`` (0 = all) starts N ranks itself, as processes (default) or as threads of this
process (``--launch threads``).  The loop per optimizer step is the reference's: (checkpoint, evaluation,)
grad-accumulation micro-steps, LR schedule, update, one host synchronisation, logging (train.cpp:512-590).
"""
from __future__ import annotations

import os
import sys
import time
from typing import Optional

import torch

from ..training.config import TrainingConfig, parse_training_config


class OutlierDetector:
    """z-score of a value against a sliding window (100 steps), as used for loss / gradient-norm monitoring."""

    def __init__(self, window: int = 100):
        self.window, self.values = window, []

    def add(self, v: float) -> float:
        z = 0.0
        if len(self.values) >= 10:
            m = sum(self.values) / len(self.values)
            var = sum((x - m) ** 2 for x in self.values) / len(self.values)
            z = (v - m) / (var ** 0.5 + 1e-12)
        self.values.append(v)
        if len(self.values) > self.window:
            self.values.pop(0)
        return z

    def state(self):
        return list(self.values)

    def restore(self, values):
        self.values = list(values)[-self.window:]


class _SyntheticLoader:
    """Uniform-random tokens with the DataLoader interface (benchmarks and smoke runs without token files)."""

    def __init__(self, vocab, seq_len, seed, rank, world):
        self.vocab, self.seq_len = vocab, seq_len
        self.gen = torch.Generator().manual_seed(seed * 1000 + rank)
        self.num_files, self.num_tokens, self.num_chunks = 0, 1 << 40, 1 << 30
        self._epoch = 0

    def load_batch(self, x, y):
        t = torch.randint(0, self.vocab, (x.shape[0], self.seq_len + 1), generator=self.gen, dtype=torch.int32)
        x.copy_(t[:, :-1])
        y.copy_(t[:, 1:])

    def has_next(self, n=1):
        return True

    def advance_epoch(self):
        self._epoch += 1

    def epoch(self):
        return self._epoch

    def progress(self):
        return 0.0

    def get_state(self):
        return {"seed": 0, "epoch": self._epoch, "file_index": 0, "chunk_index": 0, "file_name": ""}

    def set_state(self, *a):
        pass


def _resolve_continue(cfg: TrainingConfig):
    """-> (checkpoint root directory, step) or (None, -1)."""
    from ..training import checkpoint as ck
    c = cfg.continue_from_checkpoint
    if c is None:
        return None, -1
    if c == "latest":
        return cfg.checkpoint_dir, ck.find_latest_checkpoint(cfg.checkpoint_dir)
    if c.isdigit():
        return cfg.checkpoint_dir, int(c)
    base = os.path.basename(os.path.normpath(c))
    if base.startswith("step_") and os.path.exists(os.path.join(c, "checkpoint.json")):
        return os.path.dirname(os.path.normpath(c)), int(base[5:])
    return c, ck.find_latest_checkpoint(c)


def run_training(cfg: TrainingConfig, argv=None) -> dict:
    """Executed by every rank.  Returns the last step's metrics."""
    from .. import api
    from ..config import create_config_from_name, load_transformer_config
    from ..training import checkpoint as ck
    from ..training.dataloader import DataLoader
    from ..training.logging import TrainingRunLogger
    from ..training.schedule import make_schedule
    from ..utils import sol
    from ..utils.gpu_info import get_gpu_name
    from ..utils.safetensors import resolve_model_dir

    opts = cfg.to_options()
    model_dir: Optional[str] = None
    if cfg.from_scratch:
        try:
            mcfg = create_config_from_name(cfg.model, cfg.model_dtype)
        except ValueError:
            mcfg = load_transformer_config(resolve_model_dir(cfg.model), cfg.model_dtype)
    else:
        model_dir = resolve_model_dir(cfg.model)
        mcfg = load_transformer_config(model_dir, cfg.model_dtype)
    trainer = api.LLMQTrainer(ngpu=None, config=mcfg, options=opts, batch_size=cfg.batch_size, seq_len=cfg.seq_len,
                              grad_accum=cfg.grad_accumulation, memcpy_all_gather=cfg.memcpy_all_gather, memcpy_send_recv=cfg.memcpy_send_recv)
    rank, world = trainer.rank, trainer.world_size
    B, T, GA = cfg.batch_size, cfg.seq_len, cfg.grad_accumulation

    if cfg.synthetic_data:
        train_loader = _SyntheticLoader(mcfg.vocab_size, T, cfg.train_seed, rank, world)
        eval_loader = _SyntheticLoader(mcfg.vocab_size, T, cfg.eval_seed + 7, rank, world)
    else:
        train_loader = DataLoader(cfg.train_file, T, cfg.train_seed, rank, world)
        try:
            eval_loader = DataLoader(cfg.eval_file, T, cfg.eval_seed, rank, world)
        except FileNotFoundError:
            eval_loader = None
    # The tokenizer's vocabulary may be smaller than the model's (implicit padding), never larger: ids beyond the embedding
    # table would be out-of-bounds reads and writes on the device (train.cpp:429-439 refuses the same way).
    for what, loader in (("training", train_loader), ("validation", eval_loader)):
        lv = int(getattr(loader, "vocab_size", 0) or 0) if loader is not None else 0
        if lv > mcfg.vocab_size:
            raise ValueError(f"model vocab size {mcfg.vocab_size} does not match {what} data vocab size {lv}")
    step_tokens = B * T * GA * world
    steps = cfg.steps if cfg.steps > 0 else max(1, cfg.epochs * (train_loader.num_tokens // step_tokens))

    logger = TrainingRunLogger(cfg.log_file, callback=_wandb_callback(cfg) if (cfg.use_wandb and rank == 0) else None,
                               verbosity=cfg.verbosity, rank=rank, final_step=steps)
    logger.log_cmd(argv if argv is not None else sys.argv)
    logger.log_options({k: v for k, v in vars(cfg).items()})
    if trainer.device.type == "cuda":
        names = trainer.comm.host_gather((get_gpu_name(trainer.device.index), torch.cuda.get_device_properties(trainer.device).total_memory))
        for r, (n, mem) in enumerate(names or []):
            logger.log_gpu_model(r, n, mem)
    gpu_name = get_gpu_name(trainer.device.index or 0) if trainer.device.type == "cuda" else "NVIDIA B200"
    ns_spec = sol.estimate_speed_of_light(mcfg, T, opts.model_type or mcfg.dtype, opts.matmul_dtype(), world, gpu_name)
    logger.log_sol_estimate(ns_spec, spec_peak_tflops=(sol.get_gpu_spec(gpu_name) or {}).get("bf16", 0.0))
    if not cfg.synthetic_data:
        logger.log_dataset(train_loader, eval_loader)

    loss_mon, norm_mon = OutlierDetector(), OutlierDetector()
    start_step = 0
    root, ck_step = _resolve_continue(cfg)
    if root is not None:
        if ck_step < 0:
            raise FileNotFoundError(f"no checkpoint found in {root}")
        meta = trainer.load_checkpoint(root, ck_step)
        start_step = int(meta["run"]["step"])
        loss_mon.restore(meta["run"].get("past_losses", []))
        norm_mon.restore(meta["run"].get("past_norms", []))
        dl = meta.get("data-loader") or {}
        if dl and not cfg.new_data and not cfg.synthetic_data:
            train_loader.set_state(dl["seed"], dl["epoch"], dl["file_index"], dl["chunk_index"])
            if dl.get("file_name") and os.path.basename(dl["file_name"]) != os.path.basename(train_loader.current_file):
                raise RuntimeError(f"data-loader state refers to {dl['file_name']}, but the loader is at {train_loader.current_file}")
        logger.log_message(start_step, f"continuing from checkpoint {root} step {ck_step}")
    elif cfg.from_scratch:
        trainer.init_weights()
    else:
        trainer.import_weights(model_dir)
    logger.log_allocator(trainer.get_allocator_info(0), rank)
    if cfg.debug_log_allocations > 0 and getattr(trainer, "model", None) is not None:
        from ..utils.memory import large_tensors
        for name, shape, mib, where in large_tensors(trainer.model, cfg.debug_log_allocations):
            logger.log_message(start_step, f"allocation {name} {tuple(shape)} {mib:.0f} MiB ({where})")

    schedule = make_schedule(cfg.lr_schedule, cfg.learning_rate, steps, cfg.warmup_steps, cfg.final_lr_fraction, cfg.cooldown_steps)
    pin = trainer.device.type == "cuda"
    x = torch.zeros(B, T, dtype=torch.int32, pin_memory=pin)
    y = torch.zeros(B, T, dtype=torch.int32, pin_memory=pin)

    def evaluate(step):
        if eval_loader is None:
            return
        t0 = time.time()
        if not cfg.synthetic_data:
            eval_loader.set_state(cfg.eval_seed, 0, 0, 0)
        tot, tot1k, n = 0.0, 0.0, 0
        while n < cfg.eval_num_steps and eval_loader.has_next(B):
            eval_loader.load_batch(x, y)
            l, l1k = trainer.validate(x, y)
            tot, tot1k, n = tot + l, tot1k + l1k, n + 1
        if n:
            logger.log_eval(step, n * B * T * world, (time.time() - t0) * 1e3, tot / n, tot1k / n)

    def save(step):
        extra = {"data-loader": train_loader.get_state(), "run": {"past_losses": loss_mon.state(), "past_norms": norm_mon.state()}}
        trainer.save_checkpoint(cfg.checkpoint_dir, step, extra)
        if cfg.ckpt_keep_n > 0 and rank == 0:
            ck.clean_old_checkpoints(cfg.checkpoint_dir, cfg.ckpt_keep_n, cfg.ckpt_major)

    res = {}
    for step in range(start_step, steps):
        if cfg.ckpt_interval > 0 and step % cfg.ckpt_interval == 0 and step > start_step and cfg.save_training_state:
            save(step)
        if cfg.eval_every > 0 and step % cfg.eval_every == 0 and step > start_step:
            evaluate(step)
        t0 = time.time()
        for _ in range(GA):
            if not train_loader.has_next(B):
                train_loader.advance_epoch()
            train_loader.load_batch(x, y)
            trainer.step(x, y, cfg.z_loss)
        lr = schedule.eval(step)
        if cfg.log_gpu_util > 0 and step % cfg.log_gpu_util == 0 and trainer.device.type == "cuda":
            for info in trainer.get_gpu_info():
                logger.log_gpu_state(step, rank, info)
        res = trainer.update(lr, cfg.beta_1, cfg.beta_2, step + 1, cfg.weight_decay, cfg.grad_clip, cfg.adam_epsilon)
        ms = (time.time() - t0) * 1e3
        zl, zn = loss_mon.add(res["loss"]), norm_mon.add(res["norm"])
        if abs(zl) > 10 or abs(zn) > 10:
            logger.log_message(step, f"outlier detected: loss z-score {zl:.1f}, norm z-score {zn:.1f}")
        logger.log_step(step, step_tokens, ms, res["norm"], res["loss"], res["loss_1k"], res["z_max"], res["z_mean"], lr)
        if cfg.debug_time_breakdown and res.get("time_breakdown"):
            logger.log_time_breakdown(step, res["time_breakdown"])
        if cfg.debug_log_abs_max > 0 and step % cfg.debug_log_abs_max == 0 and getattr(trainer, "model", None) is not None:
            logger.log_abs_maxes(step, trainer.model.abs_maxes())
    evaluate(steps)
    if cfg.save_training_state:
        save(steps)
    trainer.export_model(cfg.out_dir)
    logger.close()
    trainer.comm.barrier()
    return res


def _child(rank: int, world: int, port: int, cfg: TrainingConfig, argv):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    run_training(cfg, argv)


def _wandb_callback(cfg, wandb=None):
    """Live export (``--use-wandb``): every log line goes to a Weights & Biases run as it is written, with the same
    mapping as the offline exporter (role of ``make_wandb_log_callback`` in the reference's binding/python/training.py)."""
    if wandb is None:
        try:
            import wandb
        except ImportError as e:
            raise RuntimeError("--use-wandb needs the wandb package; export the log file later with pyllmq-export-wandb instead") from e
    from ..scripts.export_wandb import make_wandb_log_callback
    return make_wandb_log_callback(wandb.init(project=cfg.wandb_project, name=cfg.wandb_name or cfg.name))


def main(argv=None) -> int:
    cfg = parse_training_config(argv)
    env_world = int(os.environ.get("WORLD_SIZE", os.environ.get("OMPI_COMM_WORLD_SIZE", "1")))
    n = cfg.gpus if cfg.gpus > 0 else max(1, torch.cuda.device_count())
    if env_world > 1 or n == 1:
        run_training(cfg, argv)
        return 0
    if cfg.launch == "threads":
        from ..parallel.threads import run_in_threads
        run_in_threads(n, lambda comm_env: run_training(cfg, argv))
        return 0
    import socket
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.start_processes(_child, args=(n, port, cfg, argv), nprocs=n, start_method="spawn")
    return 0


if __name__ == "__main__":
    sys.exit(main())
