"""Weights & Biases logger (reference: train/callbacks/wandb_logger.py:18-125): rank 0 only, optional
cancel-by-tag polling; a missing ``wandb`` package turns the callback into a warning."""
from __future__ import annotations

import logging
from typing import Any, Dict, Optional

from .base import Callback

log = logging.getLogger(__name__)


class WandBCallback(Callback):
    def __init__(self, project: str = "nanopsyche", entity: Optional[str] = None, group: Optional[str] = None,
                 name: Optional[str] = None, tags: Optional[list] = None, notes: Optional[str] = None,
                 cancel_check_interval: float = 300, *, config: Optional[dict] = None,
                 cancel_tags: Optional[list] = None, enabled: bool = True):
        """Arguments in the reference's order (train/callbacks/wandb_logger.py:30-39); ``cancel_check_interval`` is
        in seconds, as there: the run's tags are looked up at most that often."""
        self.group, self.notes = group, notes       # passed to wandb.init like the reference does
        self._last_cancel_check = 0.0
        self.project, self.name, self.config, self.entity, self.tags = project, name, config, entity, tags
        self.cancel_tags = cancel_tags or ["cancel", "canceled", "cancelled"]
        self.cancel_check_interval = cancel_check_interval
        self.enabled = enabled
        self._run = None
        self._wandb = None

    def pre_train(self, trainer: Any) -> None:
        if not self.enabled or not getattr(trainer, "is_main", True):
            return
        try:
            import wandb
        except ImportError:
            log.warning("wandb is not installed; WandBCallback disabled")
            self.enabled = False
            return
        self._wandb = wandb
        self._run = wandb.init(project=self.project, name=self.name, config=self.config, entity=self.entity,
                               tags=self.tags, group=self.group, notes=self.notes)

    def log_metrics(self, metrics: Dict[str, Any], step: int, trainer: Any) -> None:
        if self._run is not None:
            self._run.log(metrics, step=step)

    def post_step(self, trainer: Any) -> None:
        import time

        if self._run is None or time.monotonic() - self._last_cancel_check < self.cancel_check_interval:
            return
        self._last_cancel_check = time.monotonic()
        try:
            api_run = self._wandb.Api().run(self._run.path)
            if any(t.lower() in self.cancel_tags for t in api_run.tags):
                trainer.request_stop("cancelled by W&B tag")
        except Exception:  # noqa: BLE001
            pass

    def close(self, trainer: Any) -> None:
        if self._run is not None:
            self._run.finish()
            self._run = None
