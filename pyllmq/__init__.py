"""Drop-in import name for scripts written against the reference's ``pyllmq`` package: everything is re-exported
from ``llmq_b200`` (src/binding/python/__init__.py of the reference exposes the same names)."""
from llmq_b200.api import Config, LLMQTrainer, get_num_gpus  # noqa: F401
from llmq_b200.options import LLamaOptions  # noqa: F401
from llmq_b200.training.checkpoint import (clean_old_checkpoints, find_latest_checkpoint, get_all_checkpoints,  # noqa: F401
                                           get_checkpoint_path)
from llmq_b200.training.dataloader import DataLoader  # noqa: F401
from llmq_b200.training.logging import LogVerbosity, TrainingRunLogger  # noqa: F401
from llmq_b200.utils.gpu_info import GPUUtilInfo  # noqa: F401

from . import training  # noqa: F401,E402
from .training import CosineLRSchedule, TrainingConfig, add_training_args, training_logger_context  # noqa: F401,E402

__version__ = "0.1.0"
