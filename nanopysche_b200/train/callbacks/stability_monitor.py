"""Loss / gradient-norm spike detector (reference: train/callbacks/stability_monitor.py:18-87):
a value further than ``threshold`` standard deviations from the rolling mean counts as a spike."""
from __future__ import annotations

from collections import deque
from typing import Any, Optional

from .base import Callback


class StabilityMonitorCallback(Callback):
    def __init__(self, window_size: int = 128, threshold: float = 10.0,
                 metrics: tuple = ("train/CE loss", "optim/total grad norm"), *,
                 threshold_std: Optional[float] = None, metric_name: Optional[str] = None):
        """``threshold_std`` / ``metric_name``: the reference's names (train/callbacks/stability_monitor.py) for the
        threshold and for watching a single metric."""
        if threshold_std is not None:
            threshold = threshold_std
        if metric_name is not None:
            metrics = (metric_name,)
        if isinstance(metrics, str):        # the reference's third positional argument is one metric name
            metrics = (metrics,)
        self.window_size, self.threshold, self.metrics = window_size, threshold, tuple(metrics)
        self._hist = {m: deque(maxlen=window_size) for m in metrics}
        self._total_spikes = 0

    def _is_spike(self, name: str, v: float) -> bool:
        h = self._hist[name]
        spike = False
        if len(h) >= 8:
            mean = sum(h) / len(h)
            std = (sum((x - mean) ** 2 for x in h) / len(h)) ** 0.5
            spike = std > 0 and abs(v - mean) > self.threshold * std
        h.append(v)
        return spike

    def post_step(self, trainer: Any) -> None:
        score = 0
        for m in self.metrics:
            v = trainer.peek_metric(m) if hasattr(trainer, "peek_metric") else None
            if v is not None and self._is_spike(m, float(v)):
                score += 1
        self._total_spikes += score
        trainer.record_metric("spike/SpikeScore", score)
        trainer.record_metric("spike/SpikeScore (total)", self._total_spikes)
