"""``pyllmq.training`` names (src/binding/python/training.py of the reference)."""
import contextlib

from llmq_b200.training.config import TrainingConfig, add_training_args  # noqa: F401
from llmq_b200.training.logging import LogVerbosity, TrainingRunLogger
from llmq_b200.scripts.export_wandb import log_line_to_wandb, make_wandb_log_callback  # noqa: F401
from llmq_b200.training.schedule import CosineLRSchedule  # noqa: F401


@contextlib.contextmanager
def training_logger_context(config, callback=None):
    """Opens the run's JSON log, writes the option block, and closes the file on exit.  With ``config.use_wandb`` (and
    no callback of the caller's own) every line also goes to a Weights & Biases run."""
    if callback is None and getattr(config, "use_wandb", False):
        import wandb
        callback = make_wandb_log_callback(wandb.init(project=getattr(config, "wandb_project", "LLMQ") or "LLMQ",
                                                      name=getattr(config, "wandb_name", "") or getattr(config, "name", None)))
    logger = TrainingRunLogger(config.log_file, callback=callback, verbosity=LogVerbosity(getattr(config, "verbosity", 0)))
    try:
        logger.log_options({k: v for k, v in vars(config).items()})
        yield logger
    finally:
        logger.close()
