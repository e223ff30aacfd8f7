"""``pyllmq.scripts``: the command-line tools under their reference module paths (``pyllmq.scripts.train`` ...)."""
import importlib
import sys

for _name in ("train", "demo", "tokenize_data", "export_wandb", "watch_wandb", "plot_training_run"):
    _mod = importlib.import_module(f"llmq_b200.scripts.{_name}")
    sys.modules[f"{__name__}.{_name}"] = _mod
    globals()[_name] = _mod
