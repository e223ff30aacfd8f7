"""``pyllmq-plot``: loss / gradient-norm / throughput curves of one or more run logs, written to a PNG file
(headless Agg backend; the reference's script opens a window instead)."""
from __future__ import annotations

import argparse

from .export_wandb import read_log


def main(argv=None) -> int:
    p = argparse.ArgumentParser()
    p.add_argument("log_files", nargs="+")
    p.add_argument("--out", default="training_run.png")
    a = p.parse_args(argv)
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
    fig, ax = plt.subplots(1, 3, figsize=(15, 4))
    for path in a.log_files:
        e = read_log(path)
        st = [x for x in e if x.get("log") == "step"]
        ev = [x for x in e if x.get("log") == "eval"]
        ax[0].plot([x["step"] for x in st], [x["loss"] for x in st], label=path)
        if ev:
            ax[0].plot([x["step"] for x in ev], [x["loss"] for x in ev], "o--", label=path + " (eval)")
        ax[1].plot([x["step"] for x in st], [x["norm"] for x in st])
        ax[2].plot([x["step"] for x in st], [1000.0 * x["step_tokens"] / max(x["duration_ms"], 1e-9) for x in st])
    for a_, t in zip(ax, ("loss", "gradient norm", "tokens / s")):
        a_.set_title(t)
        a_.set_xlabel("step")
    ax[0].legend(fontsize=6)
    fig.tight_layout()
    fig.savefig(a.out, dpi=120)
    print("wrote", a.out)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
