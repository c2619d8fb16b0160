"""Throughput / MFU monitor (reference: train/callbacks/speed_monitor.py:20-166). Same metric names;
records on every rank (the metric bus averages), and the peak table holds dense bf16 figures.

Two things differ from the reference. (1) On a GPU a step's duration is the time between two CUDA events recorded around
it, read one step later (the events of the previous step have completed by then, so nothing stalls): the host runs
ahead of the device, and host wall-clock per step would report the launch time. (2) The per-device figures divide by
what one device does: tokens per step over the world size for tokens/s, and ``6 x local parameters x tokens of this
replica / context-parallel degree`` for FLOPs; with the global token count against one device's peak, as in the
reference, an 8-GPU run reports eight times its MFU."""
from __future__ import annotations

import time
from typing import Any, Optional

import torch

from .base import Callback

_GPU_PEAK_FLOPS = {"NVIDIA B200": 2.25e15, "NVIDIA H200": 989e12, "NVIDIA H100": 989e12, "NVIDIA A100": 312e12,
                   "NVIDIA A10G": 125e12, "Tesla T4": 65e12}
_DEFAULT_PEAK_FLOPS = 312e12


def _get_device_peak_flops(device: torch.device) -> float:
    if device.type != "cuda" or not torch.cuda.is_available():
        return _DEFAULT_PEAK_FLOPS
    name = torch.cuda.get_device_name(device)
    for k, v in _GPU_PEAK_FLOPS.items():
        if k in name:
            return v
    return _DEFAULT_PEAK_FLOPS


class SpeedMonitorCallback(Callback):
    def __init__(self, device: Optional[torch.device] = None, batch_size: Optional[int] = None, window_size: int = 100):
        self._device, self._batch_size, self._window_size = device, batch_size, window_size
        self._step_start = self._data_load_start = self._data_load_end = 0.0
        self._total_tokens, self._total_flops, self._total_step_time = 0, 0.0, 0.0
        self._win: list[tuple[float, int, float]] = []
        self._peak_flops: Optional[float] = None
        self._num_params: Optional[int] = None
        self._events: list = []          # (start, end) CUDA events of steps whose duration has not been read yet
        self._ev_start = None
        self._last_device_time: Optional[float] = None

    def _ensure_initialized(self, trainer: Any) -> None:
        if self._peak_flops is not None:
            return
        if self._device is None:
            self._device = getattr(trainer, "device", torch.device("cpu"))
        if self._batch_size is None:
            self._batch_size = getattr(trainer, "tokens_per_step", None) or getattr(trainer.config,
                                                                                    "global_batch_size", 1)
        self._peak_flops = _get_device_peak_flops(self._device)

    def pre_load_batch(self, trainer: Any) -> None:
        self._ensure_initialized(trainer)
        self._data_load_start = time.perf_counter()

    def pre_step(self, trainer: Any, batch: Any) -> None:
        self._data_load_end = time.perf_counter()
        self._step_start = time.perf_counter()
        if self._device is not None and self._device.type == "cuda" and torch.cuda.is_available():
            self._ev_start = torch.cuda.Event(enable_timing=True)
            self._ev_start.record()

    def _device_step_time(self) -> Optional[float]:
        """Seconds of the most recent step whose events have completed (None before the first one has)."""
        if self._ev_start is not None:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            self._events.append((self._ev_start, end))
            self._ev_start = None
        while len(self._events) > 1 or (self._events and self._events[0][1].query()):
            a, b = self._events.pop(0)
            b.synchronize()              # an older step: already complete or about to be
            self._last_device_time = a.elapsed_time(b) / 1e3
        return self._last_device_time

    def post_step(self, trainer: Any) -> None:
        self._ensure_initialized(trainer)
        if self._step_start == 0.0:
            return
        step_time = time.perf_counter() - self._step_start
        if self._device is not None and self._device.type == "cuda" and torch.cuda.is_available():
            dev_t = self._device_step_time()
            if dev_t is not None:
                step_time = max(dev_t, 1e-9)
        if step_time <= 0:
            return
        data_t = max(self._data_load_end - self._data_load_start, 0.0)
        world = max(int(getattr(trainer, "world_size", 1) or 1), 1)
        tokens, flops = self._batch_size / world, self._estimate_flops(trainer)
        self._total_tokens += self._batch_size      # whole job
        self._total_flops += flops
        self._total_step_time += step_time
        self._win.append((step_time, tokens, flops))
        if len(self._win) > self._window_size:
            self._win.pop(0)
        wt = sum(w[0] for w in self._win)
        rec = trainer.record_metric
        rec("throughput/device/TPS", tokens / step_time)
        rec("throughput/device/TPS (actual avg)", sum(w[1] for w in self._win) / wt)
        rec("throughput/device/BPS", 1.0 / step_time)
        rec("throughput/device/flopsPS", flops / step_time)
        rec("throughput/device/flopsPS (actual avg)", sum(w[2] for w in self._win) / wt)
        rec("throughput/device/MFU", 100.0 * flops / step_time / self._peak_flops)
        rec("throughput/device/MFU (actual avg)", 100.0 * sum(w[2] for w in self._win) / wt / self._peak_flops)
        rec("throughput/device/data loading (s)", data_t)
        rec("throughput/device/data loading (%)", 100.0 * data_t / step_time)
        rec("throughput/total tokens", self._total_tokens)
        rec("throughput/total petaflops", self._total_flops / 1e15)

    def _estimate_flops(self, trainer: Any) -> float:
        if self._num_params is None:
            model = getattr(trainer, "model", None)
            self._num_params = sum(p.numel() for p in model.parameters()) if model is not None else 0
        cfg = getattr(trainer, "config", None)
        replicas = max(int(getattr(cfg, "dp_world_size", 1) or 1), 1)
        cp = max(int(getattr(cfg, "cp_size", 1) or 1), 1)
        return 6.0 * self._num_params * self._batch_size / replicas / cp
