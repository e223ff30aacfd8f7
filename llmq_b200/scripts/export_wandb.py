"""``pyllmq-wandb``: replays a JSON run log into Weights & Biases (offline-friendly: needs the ``wandb`` package).

``log_line_to_metrics`` is the pure part (also used by the live watcher): it maps one log object to (step, metrics).
"""
from __future__ import annotations

import argparse
import json
from typing import Optional, Tuple


def log_line_to_metrics(obj: dict) -> Optional[Tuple[int, dict]]:
    kind = obj.get("log")
    if kind == "step":
        tps = 1000.0 * obj["step_tokens"] / obj["duration_ms"] if obj.get("duration_ms") else 0.0
        return obj["step"], {"train/loss": obj["loss"], "train/loss_1k": obj.get("loss_1k"), "train/norm": obj["norm"], "train/lr": obj.get("lr"),
                             "train/tokens_per_second": tps, "train/lse_max": obj.get("lse_max"), "train/lse_mean": obj.get("lse_mean")}
    if kind == "eval":
        return obj["step"], {"eval/loss": obj["loss"], "eval/loss_1k": obj.get("loss_1k")}
    if kind == "gpu":
        i = obj.get("id", 0)
        return obj["step"], {f"gpu{i}/power_w": (obj.get("power") or 0) / 1000.0, f"gpu{i}/clock": obj.get("clock"),
                             f"gpu{i}/temperature": obj.get("temperature"), f"gpu{i}/util": obj.get("gpu_util")}
    return None


def read_log(path: str) -> list:
    text = open(path).read().strip()
    if not text.endswith("]"):
        text = text.rstrip(",") + "\n]"          # a run that is still going (or crashed) has no closing bracket
    return json.loads(text)


def log_line_to_wandb(run, entry: dict) -> None:
    """Sends one log entry (a dict as written to the JSON log) to a Weights & Biases run."""
    if entry.get("log") == "option":
        run.config.update({entry.get("name", "option"): entry.get("value")}, allow_val_change=True)
        return
    got = log_line_to_metrics(entry)
    if got:
        run.log({k: v for k, v in got[1].items() if v is not None}, step=got[0])


def make_wandb_log_callback(run):
    """Per-line callback for ``TrainingRunLogger`` (takes the entry as a dict or as its JSON text)."""
    import json

    def callback(entry):
        log_line_to_wandb(run, json.loads(entry) if isinstance(entry, (str, bytes)) else entry)

    return callback


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description="Export a training log to wandb")
    p.add_argument("log_file")
    p.add_argument("--project", default="llmq")
    p.add_argument("--name", default=None)
    a = p.parse_args(argv)
    import wandb
    entries = read_log(a.log_file)
    config = {e["name"]: e["value"] for e in entries if e.get("log") == "option"}
    run = wandb.init(project=a.project, name=a.name, config=config)
    for e in entries:
        m = log_line_to_metrics(e)
        if m:
            run.log({k: v for k, v in m[1].items() if v is not None}, step=m[0])
    run.finish()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
