"""``pyllmq.training`` names (src/binding/python/training.py of the reference)."""
import contextlib

from llmq_b200.training.config import TrainingConfig, add_training_args  # noqa: F401
from llmq_b200.training.logging import LogVerbosity, TrainingRunLogger
from llmq_b200.training.schedule import CosineLRSchedule  # noqa: F401


@contextlib.contextmanager
def training_logger_context(config, callback=None):
    """Opens the run's JSON log, writes the option block, and closes the file on exit."""
    logger = TrainingRunLogger(config.log_file, callback=callback, verbosity=LogVerbosity(getattr(config, "verbosity", 0)))
    try:
        logger.log_options({k: v for k, v in vars(config).items()})
        yield logger
    finally:
        logger.close()
