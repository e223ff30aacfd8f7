"""The ``train`` and ``export-checkpoint`` entry points end to end on CPU with a tiny model and token files."""
import json
import math
import os

import pytest
import torch

from llmq_b200.cli import export_checkpoint, train
from llmq_b200.training import checkpoint as ck
from llmq_b200.training.config import TrainingConfig, parse_training_config
from llmq_b200.training.dataloader import write_synthetic_token_file
from llmq_b200.training.schedule import make_schedule
from llmq_b200.utils.safetensors import SafeTensorsReader


def _args(tmp_path, *extra):
    write_synthetic_token_file(str(tmp_path / "train-0.bin"), 40_000, 512, seed=0)
    write_synthetic_token_file(str(tmp_path / "eval-0.bin"), 3_000, 512, seed=1)
    return ["--model", "tiny-qwen2", "--from-scratch", "--model-dtype", "fp32", "--batch", "2", "--seq-len", "32",
            "--grad-accumulation", "2", "--steps", "6", "--lr", "1e-3", "--train-file", str(tmp_path / "train-*.bin"),
            "--eval-file", str(tmp_path / "eval-*.bin"), "--eval-every-n-steps", "4", "--eval-num-steps", "2", "--ckpt-interval", "3",
            "--name", "t", "--out-dir", str(tmp_path / "out/%n"), "--checkpoint-dir", str(tmp_path / "ckpt/%n"),
            "--log-file", str(tmp_path / "log.json"), "--gpus", "1", "--verbosity", "-2", *extra]


def test_flag_surface_and_implications():
    c = parse_training_config(["--zero-level", "3", "--recompute-block", "--matmul-dtype", "e4m3", "--name", "x", "--opt-m-dtype", "bf16"])
    assert c.shard_weights and c.shard_gradients and c.out_dir == "output/x" and c.checkpoint_dir == "ckpt/x"
    o = c.to_options()
    assert o.recompute_att and o.recompute_ffn and o.recompute_qkv and o.recompute_swiglu and o.matmul_dtype() == torch.float8_e4m3fn
    assert o.momentum_type == torch.bfloat16 and o.variance_type == torch.float32
    with pytest.raises(ValueError):
        parse_training_config(["--zero-level", "2", "--shard-weights"])
    with pytest.raises(ValueError):
        parse_training_config(["--offload-quants"])
    with pytest.raises(ValueError):
        parse_training_config(["--init-proj-to-zero"])
    for flag in ["--memcpy-all-gather", "--memcpy-send-recv", "--all-to-all-reduce", "--use-cuda-graphs", "--custom-matmul", "--write-combined",
                 "--use-zero-copy", "--offload-master", "--offload-opt-m", "--offload-opt-v", "--offload-gradients", "--offload-residual",
                 "--debug-time-breakdown", "--new-data"]:
        parse_training_config([flag])


def test_schedules():
    """Values computed by hand from the reference's formulas (schedule.h:17-53, train.cpp:563-570)."""
    s = make_schedule("cosine", 1.0, 100, warmup=10, final_lr_fraction=0.1)
    assert s.eval(0) == pytest.approx(0.1) and s.eval(9) == pytest.approx(1.0)
    # pos = (55 - 10) / 100 = 0.45 -> 0.5 cos(0.45 pi) + 0.5 = 0.578217 -> 0.9 * 0.578217 + 0.1
    assert s.eval(55) == pytest.approx(0.620396, abs=1e-5)
    # the warm-up is not subtracted from the denominator: at the last step pos = 0.9, not 1
    assert s.eval(100) == pytest.approx(0.122025, abs=1e-5)
    l = make_schedule("linear", 1.0, 100, 0, 0.0)
    assert l.eval(50) == pytest.approx(0.5) and l.eval(150) == pytest.approx(0.0)
    lw = make_schedule("linear", 2.0, 50, 10, 0.5)
    assert lw.eval(30) == pytest.approx(2.0 + (1.0 - 2.0) * 20 / 50)
    # cool-down: end_steps = 80, applies for step > 80 with f = (step - 80) / 20
    w = make_schedule("wsd", 1.0, 100, 5, 1.0, cooldown=20)
    assert w.eval(50) == 1.0 and w.eval(80) == 1.0
    assert w.eval(90) == pytest.approx(1.0 - 0.5 ** 0.5) and w.eval(99) == pytest.approx(1.0 - (19 / 20) ** 0.5) and w.eval(100) == pytest.approx(0.0)
    c = make_schedule("cosine", 1.0, 100, warmup=0, final_lr_fraction=0.0, cooldown=20)
    at_end = 0.5 * math.cos(math.pi * 80 / 80) + 0.5
    assert c.eval(80) == pytest.approx(at_end) and c.eval(40) == pytest.approx(0.5)
    assert c.eval(90) == pytest.approx(at_end * (1 - 0.5 ** 0.5))
    # the Python front end's schedule divides by (max_steps - warmup)
    from llmq_b200.training.schedule import CosineLRSchedule
    py = CosineLRSchedule(1.0, 100, 10, 0.1)
    assert py.get_lr(55) == pytest.approx(0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * 0.5))) and py.get_lr(100) == pytest.approx(0.1)


def test_token_file_with_larger_vocabulary_is_refused(tmp_path):
    """Ids beyond the embedding table must never reach the kernels: the run stops before the first step."""
    args = _args(tmp_path)
    write_synthetic_token_file(str(tmp_path / "train-0.bin"), 40_000, 600, seed=0)        # tiny-qwen2 has 512 entries
    with pytest.raises(ValueError, match="vocab size"):
        train.main(args)


def test_train_resume_and_export(tmp_path):
    args = _args(tmp_path)
    res = train.main(args)
    assert res == 0
    log = json.load(open(tmp_path / "log.json"))
    kinds = {e["log"] for e in log}
    assert {"cmd", "option", "sol", "dataset", "allocator", "step", "eval"} <= kinds
    steps = [e for e in log if e["log"] == "step"]
    assert len(steps) == 6 and steps[-1]["loss"] < steps[0]["loss"] + 0.1
    ckdir = str(tmp_path / "ckpt/t")
    assert ck.get_all_checkpoints(ckdir) == [3, 6]
    out = SafeTensorsReader(str(tmp_path / "out/t"))
    assert "model.layers.1.self_attn.k_proj.bias" in out and os.path.exists(tmp_path / "out/t/config.json")
    # resume from step 3 and land on the same losses for steps 3..5
    args2 = _args(tmp_path, "--continue", "3")
    args2[args2.index("--log-file") + 1] = str(tmp_path / "log2.json")
    train.main(args2)
    steps2 = [e for e in json.load(open(tmp_path / "log2.json")) if e["log"] == "step"]
    assert [e["step"] for e in steps2] == [3, 4, 5]
    for a, b in zip(steps[3:], steps2):
        assert a["loss"] == pytest.approx(b["loss"], abs=1e-6) and a["norm"] == pytest.approx(b["norm"], rel=1e-5)
    # stand-alone export of the latest checkpoint equals the model the run wrote
    exp = export_checkpoint.export_checkpoint("tiny-qwen2", ckdir, str(tmp_path / "exp"), model_dtype="fp32")
    a, b = SafeTensorsReader(exp), SafeTensorsReader(str(tmp_path / "out/t"))
    assert sorted(a.names()) == sorted(b.names())
    for n in a.names():
        assert torch.equal(a.read(n), b.read(n)), n


def test_python_front_end_flags_and_wandb_callback():
    """Flags of the reference's Python front end (``binding/python/training.py:183-197``): ``--offload-grads``, the
    ``-q / -qq / -v`` verbosity shortcuts and live Weights & Biases logging, checked against a stand-in for wandb."""
    cfg = parse_training_config(["--from-scratch", "--synthetic-data", "--offload-grads", "-qq", "--use-wandb", "--wandb-project", "P",
                                 "--name", "r1"])
    assert cfg.offload_gradients and cfg.verbosity == -2 and cfg.use_wandb and cfg.wandb_project == "P"
    assert parse_training_config(["-q"]).verbosity == -1 and parse_training_config(["-v"]).verbosity == 1

    class Run:
        def __init__(self):
            self.logged, self.config = [], {}

        def log(self, metrics, step=None):
            self.logged.append((step, metrics))

    class Config(dict):
        def update(self, d, allow_val_change=False):
            super().update(d)

    class FakeWandb:
        def __init__(self):
            self.run = Run()
            self.run.config = Config()

        def init(self, project=None, name=None):
            self.args = (project, name)
            return self.run

    w = FakeWandb()
    cb = train._wandb_callback(cfg, wandb=w)
    assert w.args == ("P", "r1")
    cb({"log": "option", "name": "lr", "value": 1e-3})
    cb({"log": "step", "step": 4, "step_tokens": 2048, "duration_ms": 10.0, "loss": 3.0, "norm": 1.0, "lr": 1e-3})
    cb({"log": "cmd", "argv": []})
    assert w.run.config["lr"] == 1e-3 and len(w.run.logged) == 1
    step, metrics = w.run.logged[0]
    assert step == 4 and metrics["train/loss"] == 3.0 and metrics["train/tokens_per_second"] == pytest.approx(204800.0)
    assert all(v is not None for v in metrics.values())
