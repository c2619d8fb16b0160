"""GPU memory monitor (reference: train/callbacks/gpu_memory_monitor.py:16-60); reads ``total_memory``
(the reference reads a non-existent ``total_mem`` attribute)."""
from __future__ import annotations

from typing import Any, Optional

import torch

from .base import Callback


class GPUMemoryMonitorCallback(Callback):
    def __init__(self, device: Optional[torch.device] = None):
        self._device = device

    def post_step(self, trainer: Any) -> None:
        if not torch.cuda.is_available():
            return
        dev = self._device or getattr(trainer, "device", None)
        if dev is None or torch.device(dev).type != "cuda":
            return
        stats = torch.cuda.memory_stats(dev)
        total = torch.cuda.get_device_properties(dev).total_memory
        active = stats.get("active_bytes.all.peak", 0)
        reserved = stats.get("reserved_bytes.all.peak", 0)
        gib = 1024 ** 3
        rec = trainer.record_metric
        rec("gpu_memory/GPU active mem (GiB)", active / gib)
        rec("gpu_memory/GPU active mem (%)", 100.0 * active / total)
        rec("gpu_memory/GPU reserved mem (GiB)", reserved / gib)
        rec("gpu_memory/GPU reserved mem (%)", 100.0 * reserved / total)
        torch.cuda.reset_peak_memory_stats(dev)
