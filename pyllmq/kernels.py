"""``pyllmq.kernels``: the torch custom ops of ``llmq_b200.kernels_api``."""
from llmq_b200.kernels_api import *  # noqa: F401,F403
