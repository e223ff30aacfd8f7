"""Helper scripts and telemetry on CPU: log -> metrics mapping, log tailing, plotting, tokeniser writer, fake NVML."""
import json
import os

import numpy as np
import pytest

from llmq_b200.scripts import export_wandb, plot_training_run, tokenize_data, watch_wandb
from llmq_b200.training.dataloader import DataLoader
from llmq_b200.training.logging import TrainingRunLogger
from llmq_b200.utils.gpu_info import GPUUtilTracker, set_cpu_affinity


def _log(path):
    with TrainingRunLogger(str(path), verbosity=-2) as lg:
        lg.log_options({"lr": 1e-3})
        for s in range(3):
            lg.log_step(s, 1024, 10.0, 1.5, 5.0 - s, 5.0 - s, 9.0, 8.0, 1e-3)
        lg.log_eval(3, 2048, 20.0, 4.0, 4.0)
        lg.log_gpu_state(3, 0, {"power": 700000, "clock": 1500, "temperature": 60, "gpu_utilization": 99})


def test_log_export_watch_and_plot(tmp_path):
    p = tmp_path / "run.json"
    _log(p)
    entries = export_wandb.read_log(str(p))
    got = [export_wandb.log_line_to_metrics(e) for e in entries]
    steps = [g for g in got if g and "train/loss" in g[1]]
    assert len(steps) == 3 and steps[0][1]["train/tokens_per_second"] == pytest.approx(102400.0)
    assert any(g and "eval/loss" in g[1] for g in got) and any(g and "gpu0/power_w" in g[1] for g in got)
    raw = open(p).read()
    open(tmp_path / "partial.json", "w").write(raw[: raw.rfind("]")].rstrip())      # a run that is still going
    assert len(export_wandb.read_log(str(tmp_path / "partial.json"))) == len(entries)
    tail = list(watch_wandb.follow(str(p), poll_s=0.01, stop_after_idle_s=0.02))
    assert len(tail) == len(entries)
    try:
        import matplotlib  # noqa: F401
    except ImportError:
        return
    out = tmp_path / "plot.png"
    plot_training_run.main([str(p), "--out", str(out)])
    assert out.stat().st_size > 1000


def test_tokenize_files_with_masks(tmp_path):
    class Tok:
        eos_token_id, bos_token_id = 1, 2

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [3 + (ord(c) % 50) for c in text]}

        def __len__(self):
            return 64

    src = tmp_path / "pairs.jsonl"
    with open(src, "w") as f:
        for i in range(20):
            f.write(json.dumps({"prompt": "question %d" % i, "response": "answer %d" % i}) + "\n")
    files = tokenize_data.tokenize_files([str(src)], str(tmp_path / "data" / "train"), Tok(), 64, seq_len=32, masking=True)
    dl = DataLoader(files, 32, seed=0)
    x, y = np.zeros((1, 32), np.int32), np.zeros((1, 32), np.int32)
    dl.load_batch(x, y)
    assert dl.num_tokens == 20 * 32 and (y == -100).any() and (y != -100).any()
    txt = tmp_path / "doc.txt"
    txt.write_text("first document\nline two\n\nsecond document\n")
    files = tokenize_data.tokenize_files([str(txt)], str(tmp_path / "data" / "plain"), Tok(), 64)
    assert DataLoader(files, 8).num_tokens == len("first document\nline two\n") + 1 + len("second document\n") + 1
    # several tokenizer threads give the same files, document order included
    serial = tokenize_data.tokenize_files([str(src)], str(tmp_path / "w1" / "train"), Tok(), 64, seq_len=32, masking=True)
    threaded = tokenize_data.tokenize_files([str(src)], str(tmp_path / "w4" / "train"), Tok(), 64, seq_len=32, masking=True, workers=4)
    assert [open(f, "rb").read() for f in serial] == [open(f, "rb").read() for f in threaded]


class FakeNVML:
    NVML_CLOCK_SM, NVML_TEMPERATURE_GPU, NVML_TEMPERATURE_THRESHOLD_SLOWDOWN = 1, 0, 1
    NVML_PCIE_UTIL_RX_BYTES, NVML_PCIE_UTIL_TX_BYTES = 1, 0

    def __init__(self):
        self.energy = 1_000_000
        self.calls = []

    def nvmlDeviceGetHandleByIndex(self, i):
        return ("h", i)

    def nvmlDeviceGetClockInfo(self, h, t):
        return 1350

    def nvmlDeviceGetMaxClockInfo(self, h, t):
        return 1965

    def nvmlDeviceGetFanSpeed(self, h):
        raise RuntimeError("not supported")          # data-centre parts have no fan sensor

    def nvmlDeviceGetTotalEnergyConsumption(self, h):
        self.energy += 500_000
        return self.energy

    def nvmlDeviceGetPowerUsage(self, h):
        return 900_000

    def nvmlDeviceGetEnforcedPowerLimit(self, h):
        return 1_000_000

    def nvmlDeviceGetTemperature(self, h, t):
        return 61

    def nvmlDeviceGetTemperatureThreshold(self, h, t):
        return 90

    def nvmlDeviceGetUtilizationRates(self, h):
        return type("U", (), {"gpu": 98, "memory": 40})()

    def nvmlDeviceGetCurrentClocksEventReasons(self, h):
        return 0x4 | 0x20

    def nvmlDeviceGetMemoryInfo(self, h):
        return type("M", (), {"free": 10 << 30, "total": 180 << 30})()

    def nvmlDeviceGetPcieThroughput(self, h, which):
        return 1234

    def nvmlDeviceGetCpuAffinity(self, h, n):
        return [0b1] + [0] * (n - 1)


def test_gpu_tracker_against_fake_nvml(monkeypatch):
    monkeypatch.delenv("CUDA_VISIBLE_DEVICES", raising=False)
    fake = FakeNVML()
    t = GPUUtilTracker(3, nvml=fake)
    a = t.update()
    b = t.update()
    assert a.clock == 1350 and a.max_clock == 1965 and a.fan == 0 and a.power == 900_000 and a.power_limit == 1_000_000
    assert b.power > 0 and b.temperature == 61 and b.temp_slowdown == 90 and b.gpu_utilization == 98
    assert b.throttle_reason == "sw_power_cap|sw_thermal_slowdown" and b.mem_total == 180 << 30 and b.pcie_rx == 1234
    before = os.sched_getaffinity(0)
    try:
        assert set_cpu_affinity(0, nvml=fake) in (True, False)
    finally:
        os.sched_setaffinity(0, before)


def test_tokenize_named_dataset(tmp_path):
    """``--dataset``: the named presets with an injected loader and tokenizer (no hub, no network)."""
    class Tok:
        eos_token_id, bos_token_id = 1, None

        def __call__(self, text, add_special_tokens=False):
            return {"input_ids": [3 + (ord(c) % 50) for c in text]}

        def __len__(self):
            return 64

    calls = []

    def fake_load(*hub, **kw):
        calls.append((hub, kw))
        if hub[0] == "openai/gsm8k":
            rows = [{"question": "q%d" % i, "answer": "a%d" % i} for i in range(6)]
            return {"train": rows, "test": rows[:2]}
        return {"train": ({"text": "doc %03d " % i * 5} for i in range(40))}

    files = tokenize_data.generate_tokenized_dataset("gsm8k", "qwen", str(tmp_path), load_dataset=fake_load, tokenizer=Tok())
    assert [os.path.relpath(f, tmp_path) for f in files] == ["gsm8k-qwen/train.bin", "gsm8k-qwen/eval.bin"]
    assert DataLoader(files[:1], 512).num_tokens == 6 * 512 and DataLoader(files[1:], 512).num_tokens == 2 * 512    # padded to the preset's 512
    assert calls[0] == (("openai/gsm8k", "main"), {})
    spec = dict(tokenize_data.DATASETS["fineweb-1b"], eval=100, subsample=900)
    tokenize_data.DATASETS["unit-stream"] = spec
    try:
        files = tokenize_data.generate_tokenized_dataset("unit-stream", "llama", str(tmp_path), load_dataset=fake_load, tokenizer=Tok())
    finally:
        del tokenize_data.DATASETS["unit-stream"]
    assert os.path.basename(files[0]) == "eval.bin" and os.path.basename(files[1]) == "train-000.bin" and calls[1][1] == {"streaming": True}
    n_eval, n_train = DataLoader(files[:1], 8).num_tokens, DataLoader(files[1:], 8).num_tokens
    assert 0 < n_eval <= 100 and 900 <= n_eval + n_train < 900 + 41
    with pytest.raises(ValueError):
        tokenize_data.generate_tokenized_dataset("nope", "qwen", str(tmp_path), load_dataset=fake_load, tokenizer=Tok())


def test_nvtx_ranges(monkeypatch):
    """Range helper: silent on CPU devices, balanced push / pop on a CUDA device, and it switches itself off when the
    NVTX call is not available."""
    import torch
    from llmq_b200.utils import nvtx

    calls = []

    class Fake:
        @staticmethod
        def range_push(name):
            calls.append(("push", name))

        @staticmethod
        def range_pop():
            calls.append(("pop",))

    monkeypatch.setattr(nvtx, "_backend", lambda: Fake)
    monkeypatch.setitem(nvtx._state, "on", True)
    with nvtx.range("forward", torch.device("cpu")):
        pass
    assert calls == []
    with nvtx.range("forward", torch.device("cuda", 0)):
        r = nvtx.push("Layer 3")
        nvtx.pop(r)
    assert calls == [("push", "forward"), ("push", "Layer 3"), ("pop",), ("pop",)]

    class Broken:
        @staticmethod
        def range_push(name):
            raise RuntimeError("no NVTX")

    monkeypatch.setattr(nvtx, "_backend", lambda: Broken)
    with nvtx.range("update", torch.device("cuda", 0)):
        pass
    assert nvtx._state["on"] is False and nvtx.push("x") is False


def test_api_level_training_script(tmp_path):
    """scripts/train.py drives the whole run through the Python API: steps, evaluation cadence, checkpoints with
    retention, resume from the latest checkpoint, final export."""
    import json

    from llmq_b200.scripts import train as api_train
    from llmq_b200.training import checkpoint as ck
    from llmq_b200.training.dataloader import write_synthetic_token_file

    write_synthetic_token_file(str(tmp_path / "train-0.bin"), 30_000, 512, seed=0)
    write_synthetic_token_file(str(tmp_path / "eval-0.bin"), 3_000, 512, seed=1)
    base = ["--model", "tiny-qwen2", "--from-scratch", "--model-dtype", "fp32", "--batch", "2", "--seq-len", "32", "--grad-accumulation", "2",
            "--lr", "1e-3", "--train-file", str(tmp_path / "train-*.bin"), "--eval-file", str(tmp_path / "eval-*.bin"),
            "--eval-every-n-steps", "2", "--eval-num-steps", "2", "--ckpt-interval", "2", "--ckpt-keep-n", "1", "--name", "api",
            "--out-dir", str(tmp_path / "out"), "--checkpoint-dir", str(tmp_path / "ckpt"), "--log-file", str(tmp_path / "log.json"),
            "--gpus", "1", "--verbosity", "-2", "--log-gpu-util", "0"]
    assert api_train.main(base + ["--steps", "5"]) == 0
    log = json.load(open(tmp_path / "log.json"))
    steps = [e for e in log if e["log"] == "step"]
    assert [e["step"] for e in steps] == [0, 1, 2, 3, 4] and all(e["loss"] == e["loss"] for e in steps)
    assert sum(e["log"] == "eval" for e in log) >= 3                       # steps 2 and 4 and the final one
    assert ck.get_all_checkpoints(str(tmp_path / "ckpt")) == [4, 5]        # keep-n 1 removed step 2; the final state is step 5
    assert os.path.exists(tmp_path / "out" / "model.safetensors") and os.path.exists(tmp_path / "out" / "config.json")
    # resume: continues at step 5 and runs two more
    assert api_train.main(base + ["--steps", "7", "--continue"]) == 0
    log2 = json.load(open(tmp_path / "log.json"))
    assert [e["step"] for e in log2 if e["log"] == "step"] == [5, 6]
