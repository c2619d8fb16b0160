"""Interval-gated fault-tolerant checkpointer (reference: fault_tolerance/checkpoint.py:36-157).

Writes ``step_XXXXXX/rank_XXXX_{model,optimizer}.pt`` plus ``metadata.json {step, timestamp, extra}``
through a staging directory; ``resume`` restores the newest complete checkpoint and returns its
step (0 when there is none). Truncated or half-written checkpoints (no metadata, unreadable shard)
are skipped in favour of the previous one.
"""
from __future__ import annotations

import json
import os
import shutil
import threading
import time
from typing import Optional

import torch
import torch.distributed as dist


class FaultTolerantCheckpointer:
    def __init__(self, save_dir: str = "checkpoints", save_interval: int = 100, async_save: bool = True,
                 max_stale_steps: Optional[int] = None, keep_last_n: int = 3):
        """Arguments and defaults in the reference's order (fault_tolerance/checkpoint.py:56-63). ``max_stale_steps``:
        checkpoints more than this many steps behind the newest one are removed as well (``None``: only
        ``keep_last_n`` limits them; the reference stores the value and never uses it)."""
        self.save_dir, self.save_interval, self.keep_last_n, self.async_save = save_dir, save_interval, keep_last_n, \
            async_save
        self.max_stale_steps = max_stale_steps
        os.makedirs(save_dir, exist_ok=True)
        self._thread: Optional[threading.Thread] = None

    @staticmethod
    def _rank_world():
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
        return 0, 1

    def _barrier(self):
        if self._rank_world()[1] > 1:
            dist.barrier()

    def should_save(self, step: int) -> bool:
        return step > 0 and step % self.save_interval == 0

    def save(self, step, model=None, optimizer=None, extra: Optional[dict] = None, force: bool = False,
             scheduler=None) -> Optional[str]:
        """``save(step, model, optimizer)``; the reference's order ``save(model, optimizer, step, scheduler, extra)``
        (fault_tolerance/checkpoint.py) is recognised by its first argument being a module."""
        if isinstance(step, torch.nn.Module):
            ref_model, ref_opt, ref_step = step, model, optimizer
            if isinstance(extra, dict) or extra is None:
                pass
            elif scheduler is None:          # positional (model, optimizer, step, scheduler)
                scheduler, extra = extra, None
            step, model, optimizer = int(ref_step), ref_model, ref_opt
        if not force and not self.should_save(step):
            return None
        self.wait()
        rank, _ = self._rank_world()
        def cpu(obj):
            """Deep copy to host memory: the background writer must not see tensors that later steps update (an
            optimizer's state dict hands out its live moment buffers)."""
            if torch.is_tensor(obj):
                return obj.detach().to("cpu", copy=True)
            if isinstance(obj, dict):
                return {k: cpu(v) for k, v in obj.items()}
            if isinstance(obj, (list, tuple)):
                return type(obj)(cpu(v) for v in obj)
            return obj

        msd = cpu(model.state_dict())
        osd = cpu(optimizer.state_dict()) if optimizer is not None else None
        step_dir = os.path.join(self.save_dir, f"step_{step:06d}")
        tmp = os.path.join(self.save_dir, f".tmp_step_{step:06d}")

        def write():
            os.makedirs(tmp, exist_ok=True)
            torch.save(msd, os.path.join(tmp, f"rank_{rank:04d}_model.pt"))
            if osd is not None:
                torch.save(osd, os.path.join(tmp, f"rank_{rank:04d}_optimizer.pt"))

        if self.async_save and self._rank_world()[1] == 1:
            def run():
                write()
                self._publish(step, tmp, step_dir, extra)
            self._thread = threading.Thread(target=run, daemon=True)
            self._thread.start()
            return step_dir
        write()
        self._barrier()
        if rank == 0:
            self._publish(step, tmp, step_dir, extra)
        self._barrier()
        return step_dir

    def _publish(self, step, tmp, step_dir, extra):
        with open(os.path.join(tmp, "metadata.json"), "w") as f:
            json.dump({"step": step, "timestamp": time.time(), "extra": extra or {}}, f)
        if os.path.exists(step_dir):
            shutil.rmtree(step_dir)
        os.replace(tmp, step_dir)
        done = sorted(d for d in os.listdir(self.save_dir) if d.startswith("step_"))
        for d in done[:-self.keep_last_n] if self.keep_last_n else []:
            shutil.rmtree(os.path.join(self.save_dir, d), ignore_errors=True)
        if self.max_stale_steps is not None:
            for d in done:
                try:
                    if step - int(d.split("_")[1]) > self.max_stale_steps:
                        shutil.rmtree(os.path.join(self.save_dir, d), ignore_errors=True)
                except ValueError:
                    pass

    def wait(self):
        if self._thread is not None:
            self._thread.join()
            self._thread = None

    def _loadable_steps(self) -> list:
        """Steps (newest first) whose metadata and this rank's model shard both load."""
        rank, _ = self._rank_world()
        out = []
        for d in sorted((d for d in os.listdir(self.save_dir) if d.startswith("step_")), reverse=True):
            p = os.path.join(self.save_dir, d)
            if not os.path.isfile(os.path.join(p, "metadata.json")):
                continue
            try:
                with open(os.path.join(p, "metadata.json")) as f:
                    step = int(json.load(f)["step"])
                torch.load(os.path.join(p, f"rank_{rank:04d}_model.pt"), map_location="cpu", weights_only=False)
            except Exception:  # noqa: BLE001  corrupt shard: fall back to the previous checkpoint
                continue
            out.append((step, p))
        return out

    def find_latest_checkpoint(self) -> Optional[int]:
        """Step number of the newest loadable checkpoint, ``None`` without one (reference:
        fault_tolerance/checkpoint.py:124-129 returns the step, too); ``find_latest_checkpoint_dir`` gives its path."""
        path = self.find_latest_checkpoint_dir()
        return None if path is None else int(os.path.basename(path).split("_")[1])

    def find_latest_checkpoint_dir(self) -> Optional[str]:
        """Newest checkpoint that EVERY rank can load: each rank lists the steps whose own shard is intact and the
        ranks agree on the newest common one, so a truncated shard on one rank moves all ranks back together."""
        mine = self._loadable_steps()
        _, world = self._rank_world()
        if world > 1:
            lists = [None] * world
            dist.all_gather_object(lists, [s for s, _ in mine])
            common = set(lists[0]).intersection(*map(set, lists[1:]))
            mine = [(s, p) for s, p in mine if s in common]
        return mine[0][1] if mine else None

    def resume(self, model, optimizer=None, scheduler=None) -> int:
        self.wait()
        path = self.find_latest_checkpoint_dir()
        if path is None:
            return 0
        rank, _ = self._rank_world()
        model.load_state_dict(torch.load(os.path.join(path, f"rank_{rank:04d}_model.pt"), map_location="cpu",
                                         weights_only=False))
        op = os.path.join(path, f"rank_{rank:04d}_optimizer.pt")
        if optimizer is not None and os.path.exists(op):
            optimizer.load_state_dict(torch.load(op, map_location="cpu", weights_only=False))
        with open(os.path.join(path, "metadata.json")) as f:
            step = int(json.load(f)["step"])
        if scheduler is not None:
            for _ in range(step - getattr(scheduler, "last_epoch", 0)):
                scheduler.step()
        self._barrier()
        return step
