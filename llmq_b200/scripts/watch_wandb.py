"""Tails a growing JSON run log and streams new entries to wandb (live dashboard for a run started elsewhere)."""
from __future__ import annotations

import argparse
import json
import time

from .export_wandb import log_line_to_metrics


def follow(path: str, poll_s: float = 2.0, stop_after_idle_s: float = 0.0):
    """Yields parsed log objects as lines are appended."""
    pos, idle = 0, 0.0
    while True:
        with open(path) as f:
            f.seek(pos)
            chunk = f.read()
            pos = f.tell()
        got = False
        for line in chunk.splitlines():
            line = line.strip().rstrip(",")
            if line.startswith("{"):
                try:
                    yield json.loads(line)
                    got = True
                except json.JSONDecodeError:
                    pos -= len(line)            # partial line: read it again next time
        idle = 0.0 if got else idle + poll_s
        if stop_after_idle_s and idle >= stop_after_idle_s:
            return
        time.sleep(poll_s)


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("log_file")
    p.add_argument("--project", default="llmq")
    p.add_argument("--name", default=None)
    p.add_argument("--idle-exit", type=float, default=0.0)
    a = p.parse_args(argv)
    import wandb
    run = wandb.init(project=a.project, name=a.name)
    for obj in follow(a.log_file, stop_after_idle_s=a.idle_exit):
        m = log_line_to_metrics(obj)
        if m:
            run.log({k: v for k, v in m[1].items() if v is not None}, step=m[0])
    run.finish()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
