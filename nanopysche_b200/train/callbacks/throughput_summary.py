"""End-of-run throughput summary: tokens per second over the steps after a warm-up, timed between two device
synchronisations (and barriers when distributed), so that asynchronous launches cannot flatter it. The per-step
figures of ``SpeedMonitorCallback`` are host wall-clock per step as in the reference
(train/callbacks/speed_monitor.py:96-140); this callback adds the one number a benchmark run quotes."""
from __future__ import annotations

import json
import time
from typing import Any, Optional

import torch
import torch.distributed as dist

from .base import Callback


class ThroughputSummaryCallback(Callback):
    def __init__(self, warmup_steps: int = 3, label: Optional[dict] = None):
        self.warmup_steps = warmup_steps
        self.label = label or {}
        self._t0: Optional[float] = None
        self._step0 = 0
        self._tokens0 = 0
        self.summary: Optional[dict] = None

    @staticmethod
    def _fence(trainer: Any) -> float:
        if getattr(trainer, "device", torch.device("cpu")).type == "cuda":
            torch.cuda.synchronize(trainer.device)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
            if trainer.device.type == "cuda":
                torch.cuda.synchronize(trainer.device)
        return time.perf_counter()

    def post_step(self, trainer: Any) -> None:
        if self._t0 is None and trainer.step >= self.warmup_steps:
            self._t0 = self._fence(trainer)
            self._step0, self._tokens0 = trainer.step, trainer.tokens_seen

    def post_train(self, trainer: Any) -> None:
        if self._t0 is None or trainer.step <= self._step0:
            return
        dt = self._fence(trainer) - self._t0
        steps = trainer.step - self._step0
        self.summary = dict(self.label, steps=steps, warmup=self._step0, ms_per_step=1e3 * dt / steps,
                            tokens_per_s=(trainer.tokens_seen - self._tokens0) / dt,
                            world=getattr(trainer, "world_size", 1))
        if device_is_cuda(trainer):
            self.summary["peak_mem_gb"] = torch.cuda.max_memory_allocated(trainer.device) / 2 ** 30
        if getattr(trainer, "is_main", True):
            print("throughput summary: " + json.dumps(self.summary), flush=True)


def device_is_cuda(trainer: Any) -> bool:
    return getattr(trainer, "device", torch.device("cpu")).type == "cuda"
