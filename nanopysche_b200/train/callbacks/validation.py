"""Periodic validation perplexity (the reference defines this inline in cli.py:560-577)."""
from __future__ import annotations

import math
from typing import Any, Callable

from .base import Callback


class ValidationCallback(Callback):
    def __init__(self, eval_fn: Callable[[], float], interval: int = 100):
        self.eval_fn, self.interval = eval_fn, interval

    def post_step(self, trainer: Any) -> None:
        if self.interval and trainer.step > 0 and trainer.step % self.interval == 0:
            ppl = float(self.eval_fn())
            trainer.record_metric("eval/perplexity", ppl)
            loss = math.log(max(ppl, 1e-12))
            if loss < getattr(trainer, "_best_val_loss", float("inf")):
                trainer._best_val_loss = loss
