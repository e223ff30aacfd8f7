"""Learning-rate schedules: cosine, linear, and "wsd" (warm-up, stable, 1 - sqrt cool-down).

Two families, like the reference:

* ``CosineSchedule`` / ``LinearSchedule`` / ``make_schedule`` follow the `train` executable (src/training/schedule.h:17-53,
  train.cpp:494-505 and :563-570): the decay position is ``(step - warmup) / decay_steps`` with ``decay_steps = steps -
  cooldown`` (the warm-up is NOT subtracted from the denominator), and the cool-down applies for ``step > end_steps`` with
  ``f = (step - end_steps) / cooldown`` and ``lr = schedule(end_steps) * (1 - sqrt(f))``.
* ``CosineLRSchedule`` follows the Python front end (src/binding/python/training.py:200-219): progress is
  ``(step - warmup) / (max_steps - warmup)``.

One deliberate deviation: warm-up is ``lr * (step + 1) / warmup`` in both families (the reference's C++ schedule uses
``step / warmup``, which spends step 0 at a learning rate of exactly zero; its Python schedule uses ``step + 1``).
"""
from __future__ import annotations

import math


class Schedule:
    def __init__(self, lr: float, steps: int, warmup: int = 0, final_lr: float = 0.0):
        self.lr, self.steps, self.warmup, self.final_lr = lr, max(1, steps), max(0, warmup), final_lr

    def _warm(self, step: int):
        if step < self.warmup:
            return self.lr * (step + 1) / self.warmup
        return None

    def eval(self, step: int) -> float:
        raise NotImplementedError

    get_lr = lambda self, step: self.eval(step)


class CosineSchedule(Schedule):
    """``steps`` = decay steps (schedule.h:20-28)."""

    def eval(self, step: int) -> float:
        w = self._warm(step)
        if w is not None:
            return w
        pos = (step - self.warmup) / self.steps
        frac = 0.5 * math.cos(pos * math.pi) + 0.5
        return frac * (self.lr - self.final_lr) + self.final_lr


class LinearSchedule(Schedule):
    """``steps`` = decay steps, position clamped to [0, 1] (schedule.h:38-47)."""

    def eval(self, step: int) -> float:
        w = self._warm(step)
        if w is not None:
            return w
        pos = min(1.0, max(0.0, (step - self.warmup) / self.steps))
        return self.lr + (self.final_lr - self.lr) * pos


class CosineLRSchedule(Schedule):
    """The Python front end's schedule: ``CosineLRSchedule(base_lr, max_steps, warmup_steps, final_lr)``."""

    def eval(self, step: int) -> float:
        w = self._warm(step)
        if w is not None:
            return w
        if self.warmup < self.steps:
            progress = (step - self.warmup) / (self.steps - self.warmup)
            return self.final_lr + (self.lr - self.final_lr) * 0.5 * (1.0 + math.cos(math.pi * progress))
        return self.final_lr


class _WithCooldown(Schedule):
    """``base`` up to and including ``end_steps``; after it ``base(end_steps) * (1 - sqrt((step - end_steps) / cooldown))``."""

    def __init__(self, base: Schedule, end_steps: int, cooldown: int):
        super().__init__(base.lr, end_steps + cooldown, base.warmup, base.final_lr)
        self.base, self.end_steps, self.cooldown = base, end_steps, cooldown

    def eval(self, step: int) -> float:
        if self.cooldown > 0 and step > self.end_steps:
            f = min(1.0, (step - self.end_steps) / self.cooldown)
            return self.base.eval(self.end_steps) * (1.0 - math.sqrt(f))
        return self.base.eval(step)


class WSDSchedule(_WithCooldown):
    """Constant after warm-up, then the 1 - sqrt tail over the last ``cooldown`` steps."""

    def __init__(self, lr, steps, warmup=0, final_lr=0.0, cooldown=0):
        cooldown = max(0, cooldown)
        super().__init__(LinearSchedule(lr, max(1, steps - cooldown), warmup, lr), steps - cooldown, cooldown)


def make_schedule(kind: str, lr: float, steps: int, warmup: int = 0, final_lr_fraction: float = 1.0, cooldown: int = 0) -> Schedule:
    """The `train` command line's schedule: ``end_steps = steps - cooldown`` decay steps of ``kind``, then the cool-down."""
    final = lr * final_lr_fraction
    kind = kind.lower()
    cooldown = max(0, cooldown)
    end_steps = steps - cooldown
    if kind == "wsd":
        return WSDSchedule(lr, steps, warmup, final, cooldown)
    base = {"cosine": CosineSchedule, "linear": LinearSchedule}[kind](lr, max(1, end_steps), warmup, final)
    return _WithCooldown(base, end_steps, cooldown) if cooldown > 0 else base
