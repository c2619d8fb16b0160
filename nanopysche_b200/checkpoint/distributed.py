"""Distributed checkpointing (reference: checkpoint/distributed.py:43-713).

On-disk layout (identical to the reference, metadata version 2):

    <save_dir>/step_{step:06d}[_{n}]/
        rank_{rank:04d}_model.pt / _optimizer.pt / _scheduler.pt / _rng.pt / _dataloader.json
        metadata.json   {step, world_size, model_keys, config, extra, ephemeral, version,
                         incremental, base_checkpoint, dataloader_state}
    <save_dir>/.tmp_*   staging directory, renamed into place

Beyond the reference: ``load()`` exists (base + delta chain, optimizer / scheduler / RNG / dataloader
state), every rank writes its shard into one shared staging directory that rank 0 renames once,
pinned staging is used only when CUDA is present and is synchronised before the write, and the
asynchronous save runs in a worker *process* fed with CPU tensors.
"""
from __future__ import annotations

import hashlib
import json
import os
import shutil
import time
from concurrent.futures import Future, ProcessPoolExecutor
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist


@dataclass
class CheckpointConfig:
    # fields and defaults of the reference (checkpoint/distributed.py:44-66): by default every tenth save is a full
    # one and the saves between them hold only the tensors that changed
    save_dir: str = "checkpoints"
    save_interval: int = 1000
    load_thread_count: int = 2
    keep_last_n: int = 3
    async_saves: bool = True
    save_overwrite: bool = False
    incremental: bool = True
    incremental_threshold: float = 0.01
    full_save_interval: int = 10
    pinned_memory: bool = True
    pinned_pool_size: int = 4
    save_dataloader_state: bool = True


@dataclass
class CheckpointMetadata:
    step: int = 0
    world_size: int = 1
    model_keys: List[str] = field(default_factory=list)
    config: Dict[str, Any] = field(default_factory=dict)
    extra: Dict[str, Any] = field(default_factory=dict)
    ephemeral: bool = False
    version: int = 2
    incremental: bool = False
    base_checkpoint: Optional[str] = None
    dataloader_state: Optional[Dict[str, Any]] = None


class PinnedMemoryStager:
    """Device -> host staging through pinned bounce buffers (plain ``.cpu()`` without CUDA).

    Every tensor of a state dict gets a pinned buffer of its own, keyed by its (nested) name and reused by later
    saves of the same model, so the asynchronous copies of one save never share a destination: tensors of equal
    shape (every layer's ``w_q``) must not alias. ``pool_size`` bounds how many *different* shapes may reuse a
    name's buffer before it is reallocated (a name whose shape changes gets a new buffer)."""

    def __init__(self, pool_size: int = 2, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.pool_size = pool_size
        self._pool: Dict[str, torch.Tensor] = {}

    def _buffer(self, name: str, t: torch.Tensor) -> torch.Tensor:
        buf = self._pool.get(name)
        if buf is None or buf.shape != t.shape or buf.dtype != t.dtype:
            buf = torch.empty(t.shape, dtype=t.dtype, pin_memory=self.enabled)
            self._pool[name] = buf
        return buf

    def stage_tensor(self, tensor: torch.Tensor) -> torch.Tensor:
        """One tensor to host memory (pinned when CUDA is present), a fresh buffer per call
        (reference: checkpoint/distributed.py:120-132)."""
        t = tensor.detach()
        if not (t.is_cuda and self.enabled):
            return t.cpu().clone()
        out = torch.empty(t.shape, dtype=t.dtype, pin_memory=True)
        out.copy_(t, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out

    def stage_state_dict(self, state_dict: Dict[str, Any], _prefix: str = "") -> Dict[str, Any]:
        sd = state_dict
        out: Dict[str, Any] = {}
        used_cuda = False
        for k, v in sd.items():
            if torch.is_tensor(v):
                v = v.detach()
                if hasattr(v, "full_tensor"):
                    v = v.to_local()
                if v.is_cuda and self.enabled:
                    out[k] = self._buffer(f"{_prefix}{k}", v).copy_(v, non_blocking=True)
                    used_cuda = True
                else:
                    out[k] = v.cpu()
            elif isinstance(v, dict):
                out[k] = self.stage_state_dict(v, f"{_prefix}{k}.")
            else:
                out[k] = v
        if used_cuda:
            torch.cuda.synchronize()
            # hand out copies: the bounce buffers are overwritten by the next save while a background writer or the
            # incremental checkpointer may still hold this one
            out = {k: (v.clone() if torch.is_tensor(v) and v.is_pinned() else v) for k, v in out.items()}
        return out


@dataclass
class SavePlan:
    keys: List[str] = field(default_factory=list)
    sizes: Dict[str, int] = field(default_factory=dict)
    total_bytes: int = 0
    # fields of the reference's plan (checkpoint/distributed.py:163-169); every rank writes its own shard here, so the
    # assignment is the identity and filled on request
    rank_assignments: Dict[int, List[str]] = field(default_factory=dict)
    created_at_step: int = -1
    param_hashes: Dict[str, str] = field(default_factory=dict)


class PlanCache:
    """Remembers the save plan of a model signature (keys + shapes) between saves."""

    def __init__(self):
        self._plans: Dict[str, SavePlan] = {}
        self._last: Optional[SavePlan] = None

    @staticmethod
    def signature(sd: Dict[str, torch.Tensor]) -> str:
        h = hashlib.sha256()
        for k, v in sd.items():
            h.update(k.encode())
            if torch.is_tensor(v):
                h.update(str(tuple(v.shape)).encode())
        return h.hexdigest()[:16]

    # step-keyed interface of the reference (checkpoint/distributed.py:185-201): the most recent plan, regardless of step
    def get_plan(self, step: Optional[int] = None) -> Optional[SavePlan]:
        return self._last

    def cache_plan(self, step: int, plan: SavePlan) -> None:
        self._last = plan

    def invalidate(self) -> None:
        """Forget every plan (the model's structure changed)."""
        self._plans.clear()
        self._last = None

    def get(self, sd: Dict[str, torch.Tensor]) -> SavePlan:
        sig = self.signature(sd)
        if sig not in self._plans:
            sizes = {k: v.numel() * v.element_size() for k, v in sd.items() if torch.is_tensor(v)}
            self._plans[sig] = SavePlan(list(sd.keys()), sizes, sum(sizes.values()))
        self._last = self._plans[sig]
        return self._plans[sig]


class IncrementalCheckpointer:
    """Delta saves: a key is written only if its sampled hash changed *and* its relative change
    exceeds ``threshold``; every ``full_save_interval``-th save is a full one."""

    def __init__(self, threshold: float = 0.01, full_save_interval: int = 10):
        self.threshold = threshold
        self.full_save_interval = full_save_interval
        self._hashes: Dict[str, str] = {}
        self._prev: Dict[str, torch.Tensor] = {}

    def compute_param_hash(self, tensor: torch.Tensor) -> str:
        """Sampled hash of a tensor (reference: checkpoint/distributed.py:227-241)."""
        return self._hash(tensor)

    def is_base_checkpoint_needed(self, save_count: int, full_interval: Optional[int] = None) -> bool:
        return save_count % (full_interval or self.full_save_interval) == 0

    @staticmethod
    def _hash(t: torch.Tensor) -> str:
        f = t.detach().reshape(-1).float()
        if f.numel() == 0:
            return "0" * 16
        sample = torch.cat([f[:4], f[-4:], f.sum().reshape(1), torch.tensor([float(f.numel())])])
        return hashlib.sha256(sample.cpu().numpy().tobytes()).hexdigest()[:16]

    def compute_delta(self, state_dict: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        sd = state_dict
        delta = {}
        for k, v in sd.items():
            if not torch.is_tensor(v):
                delta[k] = v
                continue
            h = self._hash(v)
            prev = self._prev.get(k)
            changed = self._hashes.get(k) != h
            if changed and prev is not None and prev.shape == v.shape:
                rel = (v.float() - prev.float()).abs().max() / (prev.float().abs().max() + 1e-8)
                changed = bool(rel >= self.threshold)
            if changed or prev is None:
                delta[k] = v
                self._hashes[k] = h
                self._prev[k] = v.detach().clone()
        return delta

    def mark_full(self, sd: Dict[str, torch.Tensor]):
        for k, v in sd.items():
            if torch.is_tensor(v):
                self._hashes[k] = self._hash(v)
                self._prev[k] = v.detach().clone()

    def should_save_full(self, save_count: int) -> bool:
        return save_count % self.full_save_interval == 0


class DataloaderStateTracker:
    def __init__(self):
        self.epoch = 0
        self.batches_seen = 0
        self.samples_seen = 0
        self.extra: Dict[str, Any] = {}

    def update(self, batch_size: Optional[int] = None, **fields):
        """``update()`` / ``update(batch_size)``: count one batch. ``update(key=value, ...)`` (the reference's form,
        checkpoint/distributed.py:309-312: current file, shard index, loader RNG state, ...): keep the fields in
        ``extra`` without counting; both together do both."""
        if fields:
            self.extra.update(fields)
            if batch_size is None:
                return
        self.batches_seen += 1
        self.samples_seen += 1 if batch_size is None else batch_size

    def get_state(self) -> Dict[str, Any]:
        import copy as _copy

        return _copy.deepcopy(self.state_dict())

    def save(self, path) -> None:
        tmp = f"{path}.tmp"
        with open(tmp, "w") as f:
            json.dump(self.state_dict(), f)
        os.replace(tmp, path)

    def load(self, path) -> None:
        if os.path.exists(path):
            with open(path) as f:
                self.load_state_dict(json.load(f))

    def new_epoch(self):
        self.epoch += 1

    def state_dict(self) -> Dict[str, Any]:
        return {"epoch": self.epoch, "batches_seen": self.batches_seen, "samples_seen": self.samples_seen,
                "extra": self.extra}

    def load_state_dict(self, sd: Dict[str, Any]):
        self.epoch = sd.get("epoch", 0)
        self.batches_seen = sd.get("batches_seen", 0)
        self.samples_seen = sd.get("samples_seen", 0)
        self.extra = sd.get("extra", {})


def _write_rank_files(tmp_dir: str, rank: int, payload: Dict[str, Any]) -> str:
    os.makedirs(tmp_dir, exist_ok=True)
    pre = os.path.join(tmp_dir, f"rank_{rank:04d}_")
    for name in ("model", "optimizer", "scheduler", "rng"):
        if payload.get(name) is not None:
            torch.save(payload[name], pre + name + ".pt")
    if payload.get("dataloader") is not None:
        with open(pre + "dataloader.json", "w") as f:
            json.dump(payload["dataloader"], f)
    return tmp_dir


def _async_save_worker(tmp_dir: str, step_dir: str, rank: int, payload: Dict[str, Any],
                       metadata: Optional[Dict[str, Any]], single_rank: bool) -> str:
    """Runs in the worker process: write this rank's files; a single-rank job also publishes."""
    _write_rank_files(tmp_dir, rank, payload)
    if single_rank:
        if metadata is not None:
            with open(os.path.join(tmp_dir, "metadata.json"), "w") as f:
                json.dump(metadata, f, indent=2, default=str)
        if os.path.exists(step_dir):
            shutil.rmtree(step_dir)
        os.replace(tmp_dir, step_dir)
    return step_dir


class DistributedCheckpointer:
    def __init__(self, config: Optional[CheckpointConfig] = None, **kw):
        self.config = config or CheckpointConfig(**kw)
        os.makedirs(self.config.save_dir, exist_ok=True)
        self.save_dir = Path(self.config.save_dir)        # as the reference exposes it (checkpoint/distributed.py:414)
        self.stager = PinnedMemoryStager(self.config.pinned_pool_size, self.config.pinned_memory)
        self.plan_cache = PlanCache()
        self.incremental = IncrementalCheckpointer(self.config.incremental_threshold, self.config.full_save_interval)
        self.dataloader_tracker = DataloaderStateTracker()
        self._save_count = 0
        self._executor: Optional[ProcessPoolExecutor] = None
        self._pending: Optional[Future] = None

    # ------------------------------------------------------------------ helpers
    @staticmethod
    def _rank_world():
        if dist.is_available() and dist.is_initialized():
            return dist.get_rank(), dist.get_world_size()
        return 0, 1

    @staticmethod
    def _barrier():
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            dist.barrier()

    def _step_dir(self, step: int) -> str:
        base = os.path.join(self.config.save_dir, f"step_{step:06d}")
        if self.config.save_overwrite or not os.path.exists(base):
            return base
        n = 1
        while os.path.exists(f"{base}_{n}"):
            n += 1
        return f"{base}_{n}"

    def _checkpoints(self) -> List[tuple]:
        out = []
        if not os.path.isdir(self.config.save_dir):
            return out
        for d in os.listdir(self.config.save_dir):
            p = os.path.join(self.config.save_dir, d)
            if d.startswith("step_") and os.path.isfile(os.path.join(p, "metadata.json")):
                try:
                    with open(os.path.join(p, "metadata.json")) as f:
                        meta = json.load(f)
                    out.append((int(meta.get("step", 0)), os.path.getmtime(p), p, meta))
                except (OSError, ValueError):
                    continue
        return sorted(out, key=lambda t: (t[0], t[1]))

    def latest_step(self) -> Optional[int]:
        c = self._checkpoints()
        return c[-1][0] if c else None

    def _find_latest_checkpoint(self) -> Optional[str]:
        c = self._checkpoints()
        return c[-1][2] if c else None

    def _find_latest_full_checkpoint(self) -> Optional[str]:
        full = [x for x in self._checkpoints() if not x[3].get("incremental")]
        return full[-1][2] if full else None

    def _cleanup_checkpoints(self):
        """Keep the last ``keep_last_n`` durable checkpoints and everything they need to be restored: the full
        base of a retained delta and every earlier delta on the same base (``load`` replays the whole chain,
        since a delta holds only the keys that changed since that key was last written)."""
        keep = self.config.keep_last_n
        if keep is None or keep <= 0:
            return
        cps = [x for x in self._checkpoints() if not x[3].get("ephemeral")]
        retained = cps[-keep:]
        needed = set()
        for st, _, _, meta in retained:
            base = meta.get("base_checkpoint")
            if not (meta.get("incremental") and base):
                continue
            needed.add(base)
            for st2, _, p2, m2 in cps:
                if m2.get("incremental") and m2.get("base_checkpoint") == base and st2 < st:
                    needed.add(os.path.basename(p2))
        for _, _, path, _ in cps[:-keep]:
            if os.path.basename(path) in needed:
                continue
            shutil.rmtree(path, ignore_errors=True)

    def _collect(self, step, model, optimizer, scheduler, extra, ephemeral, config):
        rank, world = self._rank_world()
        if hasattr(config, "as_dict"):
            config = config.as_dict()
        elif config is not None and not isinstance(config, dict):
            config = {"repr": str(config)}
        sd = model.state_dict() if hasattr(model, "state_dict") else dict(model)
        staged = self.stager.stage_state_dict(sd)
        self.plan_cache.get(staged)
        incremental = (self.config.incremental and self._save_count > 0 and
                       not self.incremental.should_save_full(self._save_count))
        base = None
        if incremental:
            base = self._find_latest_full_checkpoint()
            incremental = base is not None
        if incremental:
            model_payload = self.incremental.compute_delta(staged)
        else:
            model_payload = staged
            if self.config.incremental:
                self.incremental.mark_full(staged)
        opt_sd = self.stager.stage_state_dict(optimizer.state_dict()) if optimizer is not None else None
        sched_sd = scheduler.state_dict() if scheduler is not None else None
        rng = {"python": torch.random.get_rng_state(),
               "cuda": torch.cuda.get_rng_state_all() if torch.cuda.is_available() else None}
        dl = self.dataloader_tracker.state_dict() if self.config.save_dataloader_state else None
        payload = {"model": model_payload, "optimizer": opt_sd, "scheduler": sched_sd, "rng": rng, "dataloader": dl}
        meta = asdict(CheckpointMetadata(step=step, world_size=world, model_keys=list(sd.keys()), config=config or {},
                                         extra=extra or {}, ephemeral=ephemeral, incremental=incremental,
                                         base_checkpoint=os.path.basename(base) if base else None,
                                         dataloader_state=dl))
        return rank, world, payload, meta

    # ------------------------------------------------------------------ save
    @staticmethod
    def _save_args(args, kw):
        """``(step, model, optimizer, scheduler, extra, ephemeral, config)`` from either calling convention: this
        package's ``save(step, model, optimizer, scheduler, extra, ephemeral, config)`` or the reference's
        ``save(model, optimizer, scheduler, step, config, extra, ephemeral)`` (checkpoint/distributed.py:444-453),
        told apart by whether the first positional argument is a module."""
        ours = ("step", "model", "optimizer", "scheduler", "extra", "ephemeral", "config")
        theirs = ("model", "optimizer", "scheduler", "step", "config", "extra", "ephemeral")
        names = theirs if (args and isinstance(args[0], torch.nn.Module)) else ours
        if len(args) > len(names):
            raise TypeError(f"save() takes at most {len(names)} positional arguments")
        vals = dict(zip(names, args))
        for k, v in kw.items():
            if k not in ours:
                raise TypeError(f"save() got an unexpected keyword argument {k!r}")
            if k in vals:
                raise TypeError(f"save() got multiple values for argument {k!r}")
            vals[k] = v
        if "model" not in vals:
            raise TypeError("save() needs a model")
        return (int(vals.get("step", 0)), vals["model"], vals.get("optimizer"), vals.get("scheduler"),
                vals.get("extra"), bool(vals.get("ephemeral", False)), vals.get("config"))

    def save(self, *args, **kw) -> Path:
        """Synchronous save; every rank must call it. ``save(step, model, optimizer=None, scheduler=None, extra=None,
        ephemeral=False, config=None)``; the reference's positional order ``save(model, optimizer, scheduler, step, ...)``
        is accepted as well."""
        step, model, optimizer, scheduler, extra, ephemeral, config = self._save_args(args, kw)
        self.wait()
        rank, world, payload, meta = self._collect(step, model, optimizer, scheduler, extra, ephemeral, config)
        step_dir = self._step_dir(step)
        if world > 1:
            names = [step_dir]
            dist.broadcast_object_list(names, src=0)
            step_dir = names[0]
        tmp_dir = os.path.join(self.config.save_dir, ".tmp_" + os.path.basename(step_dir))
        if rank == 0 and os.path.exists(tmp_dir):
            shutil.rmtree(tmp_dir)
        self._barrier()
        _write_rank_files(tmp_dir, rank, payload)
        self._barrier()
        if rank == 0:
            with open(os.path.join(tmp_dir, "metadata.json"), "w") as f:
                json.dump(meta, f, indent=2, default=str)
            if os.path.exists(step_dir):
                shutil.rmtree(step_dir)
            os.replace(tmp_dir, step_dir)
            self._cleanup_checkpoints()
        self._barrier()
        self._save_count += 1
        return Path(step_dir)

    def save_async(self, *args, **kw) -> Future:
        """Stage on the caller, write in a worker process (a process rather than a thread keeps the
        GIL free for the training loop). Multi-rank jobs publish in ``wait()``. Arguments as for ``save``."""
        step, model, optimizer, scheduler, extra, ephemeral, config = self._save_args(args, kw)
        self.wait()
        rank, world, payload, meta = self._collect(step, model, optimizer, scheduler, extra, ephemeral, config)
        step_dir = self._step_dir(step)
        tmp_dir = os.path.join(self.config.save_dir, ".tmp_" + os.path.basename(step_dir))
        if self._executor is None:
            import multiprocessing as mp

            self._executor = ProcessPoolExecutor(max_workers=1, mp_context=mp.get_context("spawn"))
        fut = self._executor.submit(_async_save_worker, tmp_dir, step_dir, rank, payload, meta if rank == 0 else None,
                                    world == 1)
        self._pending = fut
        self._pending_info = (rank, world, tmp_dir, step_dir, meta)
        self._save_count += 1
        return fut

    def wait(self):
        """Block until the outstanding asynchronous save is on disk (and published)."""
        if self._pending is None:
            return
        fut, self._pending = self._pending, None
        fut.result()
        rank, world, tmp_dir, step_dir, meta = self._pending_info
        if world > 1:
            self._barrier()
            if rank == 0:
                with open(os.path.join(tmp_dir, "metadata.json"), "w") as f:
                    json.dump(meta, f, indent=2, default=str)
                if os.path.exists(step_dir):
                    shutil.rmtree(step_dir)
                os.replace(tmp_dir, step_dir)
            self._barrier()
        if rank == 0:
            self._cleanup_checkpoints()

    def close(self):
        self.wait()
        if self._executor is not None:
            self._executor.shutdown()
            self._executor = None

    # ------------------------------------------------------------------ load
    def load(self, path: Optional[str] = None, model=None, optimizer=None, scheduler=None,
             restore_rng: bool = True, strict: bool = True) -> Dict[str, Any]:
        """Restore from ``path`` (a ``step_*`` directory or the save dir; default: the latest
        checkpoint). Applies the full base first when the checkpoint is a delta. Returns the metadata."""
        self.wait()
        if path is None or os.path.abspath(path) == os.path.abspath(self.config.save_dir):
            path = self._find_latest_checkpoint()
        elif not os.path.isfile(os.path.join(path, "metadata.json")):
            inner = DistributedCheckpointer(CheckpointConfig(save_dir=path))._find_latest_checkpoint()
            path = inner or path
        if path is None or not os.path.isfile(os.path.join(path, "metadata.json")):
            raise FileNotFoundError(f"no checkpoint found under {path or self.config.save_dir}")
        with open(os.path.join(path, "metadata.json")) as f:
            meta = json.load(f)
        rank, world = self._rank_world()
        saved_world = int(meta.get("world_size") or world)
        # Resuming on another number of ranks (pure data parallelism): the replicated model is in every rank's file,
        # the sharded optimizer state is put together from all of them (``load_state_dict_resharded``)
        src_rank = rank if rank < saved_world else rank % saved_world
        pre = os.path.join(path, f"rank_{src_rank:04d}_")

        def _load(p):
            return torch.load(p, map_location="cpu", weights_only=False)

        if model is not None:
            sd: Dict[str, Any] = {}
            if meta.get("incremental") and meta.get("base_checkpoint"):
                base = os.path.join(os.path.dirname(path), meta["base_checkpoint"])
                sd.update(_load(os.path.join(base, f"rank_{src_rank:04d}_model.pt")))
                # deltas between the base and this one, oldest first
                for st, _, p, m in self._checkpoints_in(os.path.dirname(path)):
                    if m.get("incremental") and m.get("base_checkpoint") == meta["base_checkpoint"] and \
                            st < meta["step"]:
                        sd.update(_load(os.path.join(p, f"rank_{src_rank:04d}_model.pt")))
            sd.update(_load(pre + "model.pt"))
            model.load_state_dict(sd, strict=strict)
        if optimizer is not None and saved_world != world and hasattr(optimizer, "load_state_dict_resharded"):
            optimizer.load_state_dict_resharded(
                [_load(os.path.join(path, f"rank_{i:04d}_optimizer.pt")) for i in range(saved_world)])
        elif optimizer is not None and os.path.exists(pre + "optimizer.pt"):
            optimizer.load_state_dict(_load(pre + "optimizer.pt"))
        if scheduler is not None and os.path.exists(pre + "scheduler.pt"):
            scheduler.load_state_dict(_load(pre + "scheduler.pt"))
        if restore_rng and os.path.exists(pre + "rng.pt"):
            rng = _load(pre + "rng.pt")
            torch.random.set_rng_state(rng["python"])
            if rng.get("cuda") is not None and torch.cuda.is_available():
                try:
                    torch.cuda.set_rng_state_all(rng["cuda"])
                except Exception:  # noqa: BLE001  (different GPU count)
                    pass
        if os.path.exists(pre + "dataloader.json"):
            with open(pre + "dataloader.json") as f:
                self.dataloader_tracker.load_state_dict(json.load(f))
        return meta

    @staticmethod
    def _checkpoints_in(save_dir: str):
        return DistributedCheckpointer(CheckpointConfig(save_dir=save_dir))._checkpoints()
