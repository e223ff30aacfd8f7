"""``pyllmq-train``: the training loop written against the Python API (``LLMQTrainer`` / ``DataLoader`` / logger),
the counterpart of the reference's scripts/train.py; ``python -m llmq_b200.cli.train`` is the full-featured driver."""
from ..cli.train import main

if __name__ == "__main__":
    raise SystemExit(main())
