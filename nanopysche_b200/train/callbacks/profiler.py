"""torch.profiler callback (reference: train/callbacks/profiler.py:22-174): skip/wait/warm-up/active
window, Chrome trace per rank, top-k kernel tables. The in-tree kernels show up under their own
names; the Trainer does call ``pre_step`` here, so the window actually opens."""
from __future__ import annotations

import logging
import os
from typing import Any, Optional

import torch

from .base import Callback

log = logging.getLogger(__name__)


class ProfilerCallback(Callback):
    def __init__(self, skip_first: int = 10, wait: int = 5, warmup: int = 5, active: int = 10, repeat: int = 1,
                 with_stack: bool = True, profile_memory: bool = True, enable_cuda_sync_events: bool = True,
                 output_dir: str = "profiler", profile_ranks: Optional[str] = None, *,
                 save_dir: Optional[str] = None, record_shapes: bool = False, with_flops: bool = False,
                 row_limit: int = 20):
        """Arguments and defaults in the reference's order (train/callbacks/profiler.py:39-50); ``save_dir`` is another
        name for ``output_dir``; ``enable_cuda_sync_events`` is accepted and ignored (the Kineto switch it set only
        adds synchronisation records to the trace)."""
        save_dir = save_dir or output_dir
        self.save_dir = save_dir
        self.skip_first, self.wait, self.warmup, self.active, self.repeat = skip_first, wait, warmup, active, repeat
        self.profile_ranks = profile_ranks
        self.opts = dict(with_stack=with_stack, profile_memory=profile_memory, record_shapes=record_shapes,
                         with_flops=with_flops)
        self.row_limit = row_limit
        self._prof = None
        self._first_step: Optional[int] = None
        self._done = False

    def _enabled_on(self, trainer: Any) -> bool:
        rank = getattr(trainer, "rank", 0)
        return self.profile_ranks == "all" or rank == 0

    def pre_step(self, trainer: Any, batch: Any) -> None:
        if self._done or not self._enabled_on(trainer):
            return
        if self._first_step is None:
            self._first_step = trainer.step
        rel = trainer.step - self._first_step
        start = self.skip_first + self.wait
        if rel == start and self._prof is None:
            acts = [torch.profiler.ProfilerActivity.CPU]
            if torch.cuda.is_available():
                acts.append(torch.profiler.ProfilerActivity.CUDA)
            self._prof = torch.profiler.profile(activities=acts, **self.opts)
            self._prof.__enter__()

    def post_step(self, trainer: Any) -> None:
        if self._prof is None or self._first_step is None:
            return
        rel = trainer.step - self._first_step
        if rel >= self.skip_first + self.wait + self.warmup + self.active:
            self._stop(trainer)

    def _stop(self, trainer: Any) -> None:
        prof, self._prof = self._prof, None
        self._done = True
        prof.__exit__(None, None, None)
        os.makedirs(self.save_dir, exist_ok=True)
        rank = getattr(trainer, "rank", 0)
        path = os.path.join(self.save_dir, f"rank-{rank}-step-{trainer.step}.chrome_trace.json.gz")
        try:
            prof.export_chrome_trace(path)
        except Exception as e:  # noqa: BLE001
            log.warning("could not export trace: %s", e)
        key = "self_cuda_time_total" if torch.cuda.is_available() else "self_cpu_time_total"
        log.info("\n%s", prof.key_averages().table(sort_by=key, row_limit=self.row_limit))
        self.last_trace_path = path

    def close(self, trainer: Any) -> None:
        if self._prof is not None:
            self._stop(trainer)
