"""Learning-rate schedules (reference: train/scheduler.py:20-174): plain functions of the step and
``LambdaLR`` subclasses with the same constructor arguments."""
from __future__ import annotations

import math

from torch.optim.lr_scheduler import LambdaLR


def cosine_with_warmup(step: int, warmup_steps: int, max_steps: int, min_lr: float = 0.0, max_lr: float = 1e-3):
    if step < warmup_steps:
        return max_lr * step / max(warmup_steps, 1)
    if step >= max_steps:
        return min_lr
    progress = (step - warmup_steps) / max(max_steps - warmup_steps, 1)
    return min_lr + 0.5 * (max_lr - min_lr) * (1 + math.cos(math.pi * progress))


def warmup_stable_decay(step: int, warmup_steps: int, stable_steps: int, decay_steps: int, min_lr: float = 0.0,
                        max_lr: float = 1e-3, decay_lr: float | None = None):
    total = warmup_steps + stable_steps + decay_steps
    if step < warmup_steps:
        return max_lr * step / max(warmup_steps, 1)
    if step < warmup_steps + stable_steps:
        return max_lr
    if step < total:
        p = (step - warmup_steps - stable_steps) / max(decay_steps, 1)
        return min_lr + 0.5 * (max_lr - min_lr) * (1 + math.cos(math.pi * p))
    return min_lr


def exponential_decay(step: int, warmup_steps: int, decay_rate: float = 0.999, min_lr: float = 0.0,
                      max_lr: float = 1e-3):
    if step < warmup_steps:
        return max_lr * step / max(warmup_steps, 1)
    return max(min_lr, max_lr * (decay_rate ** (step - warmup_steps)))


class CosineWithWarmup(LambdaLR):
    """Multiplier: linear warm-up to 1, cosine to ``min_lr_ratio``, flat afterwards."""

    def __init__(self, optimizer, warmup_steps: int, max_steps: int, min_lr_ratio: float = 0.1, last_epoch: int = -1):
        self.warmup_steps, self.max_steps, self.min_lr_ratio = warmup_steps, max_steps, min_lr_ratio
        super().__init__(optimizer, self._lr_lambda, last_epoch)

    def _lr_lambda(self, step: int) -> float:
        return cosine_with_warmup(step, self.warmup_steps, self.max_steps, self.min_lr_ratio, 1.0)


class WarmupStableDecay(LambdaLR):
    def __init__(self, optimizer, warmup_steps: int, stable_steps: int, decay_steps: int,
                 min_lr_ratio: float = 0.1, last_epoch: int = -1):
        self.warmup_steps, self.stable_steps, self.decay_steps = warmup_steps, stable_steps, decay_steps
        self.min_lr_ratio = min_lr_ratio
        super().__init__(optimizer, self._lr_lambda, last_epoch)

    def _lr_lambda(self, step: int) -> float:
        return warmup_stable_decay(step, self.warmup_steps, self.stable_steps, self.decay_steps, self.min_lr_ratio,
                                   1.0)
