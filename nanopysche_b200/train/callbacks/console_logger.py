"""Console logger (reference: train/callbacks/console_logger.py:19-88): glob-filtered metrics with an
ETA. Prints through ``logging`` and installs a stream handler if none is configured (the reference
logs at INFO with no handler, so nothing appears by default)."""
from __future__ import annotations

import fnmatch
import logging
import time
from typing import Any, Dict, Optional, Sequence

from .base import Callback

log = logging.getLogger("nanopsyche.train")

DEFAULT_LOG_PATTERNS = ["train/*", "optim/LR", "optim/total grad norm", "throughput/device/TPS",
                        "throughput/device/MFU", "throughput/total tokens", "gpu_memory/GPU active mem (GiB)",
                        "spike/*", "eval/*"]


class ConsoleLoggerCallback(Callback):
    def __init__(self, patterns: Optional[Sequence[str]] = None, log_interval: int = 1,
                 metrics_to_log: Optional[Sequence[str]] = None):
        """``metrics_to_log``: the reference's name for the list of metric patterns (train/callbacks/console_logger.py)."""
        self.patterns = list(patterns or metrics_to_log or DEFAULT_LOG_PATTERNS)
        self.log_interval = log_interval
        self._t0: Optional[float] = None

    def pre_train(self, trainer: Any) -> None:
        self._t0 = time.time()
        if not log.handlers and not logging.getLogger().handlers:
            h = logging.StreamHandler()
            h.setFormatter(logging.Formatter("%(asctime)s %(message)s", "%H:%M:%S"))
            log.addHandler(h)
            log.setLevel(logging.INFO)

    def log_metrics(self, metrics: Dict[str, Any], step: int, trainer: Any) -> None:
        if step % self.log_interval:
            return
        shown = {k: v for k, v in metrics.items() if any(fnmatch.fnmatch(k, p) for p in self.patterns)}
        parts = [f"{k}={v:.4g}" if isinstance(v, (int, float)) else f"{k}={v}" for k, v in sorted(shown.items())]
        eta = ""
        max_steps = getattr(trainer.config, "max_steps", 0)
        if self._t0 is not None and step > 0 and max_steps:
            rem = (time.time() - self._t0) / step * (max_steps - step)
            eta = f" eta={rem / 60:.1f}m"
        log.info("step %d/%s%s | %s", step, max_steps or "?", eta, " ".join(parts))
