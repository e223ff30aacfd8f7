"""Learning-rate schedules: cosine, linear, and "wsd" (warm-up, stable, 1 - sqrt cool-down).

Reference: src/training/schedule.h:11-53 and the cool-down logic of train.cpp:494-555.  Warm-up is
``lr * (step + 1) / warmup`` in both front-ends here (the reference's C++ and Python schedules differ by one step).
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
    def eval(self, step: int) -> float:
        w = self._warm(step)
        if w is not None:
            return w
        t = min(1.0, (step - self.warmup) / max(1, self.steps - self.warmup))
        return self.final_lr + 0.5 * (self.lr - self.final_lr) * (1.0 + math.cos(math.pi * t))


class LinearSchedule(Schedule):
    def eval(self, step: int) -> float:
        w = self._warm(step)
        if w is not None:
            return w
        t = min(1.0, (step - self.warmup) / max(1, self.steps - self.warmup))
        return self.lr + (self.final_lr - self.lr) * t


class WSDSchedule(Schedule):
    """Constant after warm-up, then an annealing tail of ``cooldown`` steps shaped like 1 - sqrt(progress)."""

    def __init__(self, lr, steps, warmup=0, final_lr=0.0, cooldown=0):
        super().__init__(lr, steps, warmup, final_lr)
        self.cooldown = max(0, cooldown)

    def eval(self, step: int) -> float:
        w = self._warm(step)
        if w is not None:
            return w
        start = self.steps - self.cooldown
        if self.cooldown > 0 and step >= start:
            t = min(1.0, (step - start + 1) / self.cooldown)
            return self.final_lr + (self.lr - self.final_lr) * (1.0 - math.sqrt(t))
        return self.lr


CosineLRSchedule = CosineSchedule


def make_schedule(kind: str, lr: float, steps: int, warmup: int = 0, final_lr_fraction: float = 1.0, cooldown: int = 0) -> Schedule:
    """``cooldown`` > 0 adds the 1 - sqrt tail to any schedule kind, like the reference CLI."""
    final = lr * final_lr_fraction
    kind = kind.lower()
    if kind == "wsd":
        return WSDSchedule(lr, steps, warmup, final if cooldown == 0 else 0.0, cooldown)
    base = {"cosine": CosineSchedule, "linear": LinearSchedule}[kind](lr, max(1, steps - cooldown), warmup, final)
    if cooldown <= 0:
        return base

    class _Tail(Schedule):
        def eval(self_inner, step):
            start = steps - cooldown
            if step < start:
                return base.eval(step)
            t = min(1.0, (step - start + 1) / cooldown)
            return base.eval(start) * (1.0 - math.sqrt(t))

    return _Tail(lr, steps, warmup, final)
