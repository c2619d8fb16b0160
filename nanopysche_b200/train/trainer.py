"""Training loop (reference: train/trainer.py:30-449).

Same public surface as the reference (``TrainingConfig``, ``Trainer(...).fit()``, ``record_metric``,
``load_checkpoint``, the metric names, the callback lifecycle) with its loop defects designed out:

* gradient accumulation is ``max(1, global_batch // (micro * seq * dp))`` with ``global_batch`` in
  tokens (a value smaller than one micro-batch of tokens is read as a number of sequences), so the
  CLI path actually trains;
* ``pre_step`` / ``post_train`` are called, metrics are reduced on *every* rank (a collective inside
  ``if is_main`` deadlocks) and every rank takes part in checkpoint saves;
* losses stay on the device: nothing calls ``.item()`` per micro-batch, values are read when metrics
  are flushed;
* with an ``ArenaAdamW`` optimizer the clip / step / zero-grad path is the fused one and the step is
  timed on the device with CUDA events.
"""
from __future__ import annotations

import logging
import math
import os
import time
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .callbacks.base import Callback

log = logging.getLogger(__name__)


@dataclass
class TrainingConfig:
    global_batch_size: int = 1024
    micro_batch_size: int = 4
    sequence_length: int = 2048
    learning_rate: float = 3e-4
    min_lr: float = 3e-5
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    warmup_steps: int = 2000
    max_steps: int = 600000
    dtype: torch.dtype = torch.bfloat16
    loss_scale: float = 1.0
    save_interval: int = 1000
    save_dir: str = "checkpoints"
    log_interval: int = 10
    dp_world_size: int = 1
    enable_hang_detection: bool = False
    enable_gradient_compression: bool = False
    compression_rank: int = 256
    vocab_size: int = 32000
    cp_size: int = 1
    pp_schedule: str = "1F1B"          # pipeline schedule when the model is a pipeline stage
    pp_microbatches: int = 0           # 0: one microbatch per pipeline rank

    @property
    def tokens_per_micro_step(self) -> int:
        return self.micro_batch_size * self.sequence_length * max(self.dp_world_size, 1)

    @property
    def gradient_accumulation_steps(self) -> int:
        g = self.global_batch_size
        if g < self.micro_batch_size * self.sequence_length:  # given in sequences
            g = g * self.sequence_length
        return max(1, g // self.tokens_per_micro_step)

    @property
    def dp_size(self) -> int:
        return self.dp_world_size


class Trainer:
    def __init__(self, config: TrainingConfig, model: nn.Module, optimizer: torch.optim.Optimizer,
                 scheduler=None, data_loader=None, callbacks: Optional[List[Callback]] = None, checkpointer=None,
                 hang_detector=None, heartbeat=None, device: Optional[torch.device] = None, status_reader=None):
        self.config = config
        self.model = model
        self.optimizer = optimizer
        self.scheduler = scheduler
        self.data_loader = data_loader
        self.callbacks = callbacks or []
        self.checkpointer = checkpointer
        self.hang_detector = hang_detector
        self.heartbeat = heartbeat
        self.step = 0
        self.tokens_seen = 0
        self._metrics: Dict[str, Any] = {}
        self._compressor = None
        self._leave_after: Optional[int] = None    # this rank's announced last step (leave_after_step)
        self._best_val_loss = float("inf")
        self._stop_reason: Optional[str] = None
        self.emergency_checkpoint_dir: Optional[str] = None
        self._data_iter = None
        self._setup_distributed(device)
        # reads the kernels' device status words ((code, kernel, block, detail, ...); code 0 = ok). The fused kernels
        # bound every wait on a peer and record a code instead of hanging; the trainer looks at it wherever it
        # synchronises with the device anyway (metric flush, checkpoint)
        self._status_reader = status_reader
        if status_reader is None and self.device.type == "cuda":
            from ..ops import _lib

            self._status_reader = _lib.status
        if config.enable_hang_detection and self.hang_detector is None:
            from ..fault_tolerance.hang_detection import HangDetector

            self.hang_detector = HangDetector()
        if config.enable_gradient_compression:
            # replaces the data-parallel gradient all-reduce (the reference constructs the compressor but never calls
            # it, train/trainer.py:112-119; here it is the gradient synchronisation of the un-sharded path)
            from ..optim.diko import DiLoCoCompressor

            if self._arena_opt or getattr(model, "_fsdp_enabled", False):
                raise ValueError("enable_gradient_compression needs un-sharded data parallelism: the parameter arena "
                                 "and FSDP reduce-scatter full-precision gradients into shards")
            self._compressed_params = [p for p in model.parameters()
                                       if p.requires_grad and not getattr(p, "_ep_sharded", False)]
            self._compressor = DiLoCoCompressor(self._compressed_params, compression_rank=config.compression_rank,
                                                group=getattr(model, "_replica_group", None))

    # ------------------------------------------------------------------ setup
    def _setup_distributed(self, device=None):
        self.rank, self.world_size = 0, 1
        if dist.is_available() and not dist.is_initialized() and "RANK" in os.environ:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
            dist.init_process_group(backend=backend)
        if dist.is_available() and dist.is_initialized():
            self.rank, self.world_size = dist.get_rank(), dist.get_world_size()
        self.is_main = self.rank == 0
        if device is not None:
            self.device = torch.device(device)
        else:
            p = next(self.model.parameters(), None)
            self.device = p.device if p is not None else torch.device("cpu")
        self._arena_opt = type(self.optimizer).__name__ == "ArenaAdamW"
        self._reducer = None           # parallel.ddp.BucketedGradReducer, built on first use
        self._pp_schedule = None       # built on the first step when the model is one stage of a pipeline

    @property
    def tokens_per_step(self) -> int:
        c = self.config
        return c.micro_batch_size * c.sequence_length * max(c.dp_world_size, 1) * c.gradient_accumulation_steps

    # ------------------------------------------------------------------ metrics bus
    def record_metric(self, name: str, value) -> None:
        self._metrics[name] = value

    def peek_metric(self, name: str):
        v = self._metrics.get(name)
        return float(v) if v is not None else None

    def check_device_status(self, where: str = "") -> None:
        """Raise if a kernel of an earlier step gave up on a bounded wait (a peer that stopped answering) or failed a
        device-side check. ``CommTimeoutError`` for timeouts, ``KernelError`` otherwise; ``fit()`` then runs the
        ``on_error`` callbacks and writes an emergency checkpoint of this rank's state."""
        if self._status_reader is None:
            return
        st = tuple(self._status_reader())
        if not st or st[0] == 0:
            return
        from ..fault_tolerance.hang_detection import CommTimeoutError
        from ..ops import _lib

        if self.device.type == "cuda":
            _lib.lib().np_status_clear()
        msg = (f"device status {st[0]} ({_lib.STATUS_NAMES.get(st[0], '?')}) kernel={st[1] if len(st) > 1 else '?'} "
               f"block={st[2] if len(st) > 2 else '?'} detail={st[3] if len(st) > 3 else '?'} at step {self.step} {where}")
        if st[0] in (1, 2):
            raise CommTimeoutError(msg)
        raise _lib.KernelError(msg)

    def _emergency_checkpoint(self) -> Optional[str]:
        """This rank's model / optimizer state written without any collective (peers may be gone):
        ``<save_dir>/emergency_step_{step:06d}/rank_{rank:04d}_{model,optimizer}.pt``."""
        try:
            d = os.path.join(self.config.save_dir, f"emergency_step_{self.step:06d}")
            os.makedirs(d, exist_ok=True)
            torch.save({k: v.detach().cpu() for k, v in self.model.state_dict().items()},
                       os.path.join(d, f"rank_{self.rank:04d}_model.pt"))
            torch.save(self.optimizer.state_dict(), os.path.join(d, f"rank_{self.rank:04d}_optimizer.pt"))
            # the same metadata from every rank (whoever writes last wins, the content is identical): makes the
            # directory loadable by DistributedCheckpointer.load, also on another number of ranks
            import json

            meta = {"step": self.step, "world_size": self.world_size, "model_keys": list(self.model.state_dict().keys()),
                    "config": {}, "extra": {"tokens_seen": self.tokens_seen, "emergency": True}, "ephemeral": False,
                    "incremental": False, "base_checkpoint": None, "dataloader_state": None}
            tmp = os.path.join(d, f".metadata.{self.rank}.tmp")
            with open(tmp, "w") as f:
                json.dump(meta, f)
            os.replace(tmp, os.path.join(d, "metadata.json"))
            return d
        except Exception as e:  # noqa: BLE001
            log.error("emergency checkpoint failed: %s", e)
            return None

    def _flush_metrics(self) -> Dict[str, float]:
        """Average the buffered metrics over all ranks (every rank must call this)."""
        self.check_device_status("(metric flush)")
        names = sorted(self._metrics)
        vals = torch.tensor([float(self._metrics[n]) for n in names], dtype=torch.float64)
        if self.world_size > 1 and dist.is_initialized():
            present = [None] * self.world_size
            dist.all_gather_object(present, names)
            common = sorted(set.intersection(*map(set, present)))
            idx = [names.index(n) for n in common]
            sub = vals[idx].to(self.device if self.device.type == "cuda" else "cpu")
            dist.all_reduce(sub)
            vals[idx] = (sub / self.world_size).cpu()
        out = {n: float(v) for n, v in zip(names, vals)}
        self._metrics = {}
        if self.is_main:
            for cb in self.callbacks:
                cb.pre_log_metrics(self)
            for cb in self.callbacks:
                cb.log_metrics(out, self.step, self)
            for cb in self.callbacks:
                cb.post_log_metrics(self)
        return out

    def get_vocab_size(self) -> int:
        """Vocabulary size for synthetic batches: the model's, else the configured one
        (reference: train/trainer.py:361-367)."""
        v = getattr(self.model, "vocab_size", None)
        if v:
            return int(v)
        emb = getattr(self.model, "embeddings", None)
        if emb is not None and hasattr(emb, "weight"):
            return int(emb.weight.shape[0])
        return int(getattr(self.config, "vocab_size", 32000) or 32000)

    def request_stop(self, reason: str = "") -> None:
        self._stop_reason = reason or "stop requested"

    def leave_after_step(self, last_step: Optional[int] = None) -> None:
        """This rank leaves the job (preemption notice, planned shrink) after completing ``last_step`` (default: the
        step that is about to run or running). Call it before that step's collectives start - from ``pre_step`` or
        earlier; the peers find the note at the top of the following step and stop there with ``PeerLeftError``
        (their ``on_error`` callbacks run and each writes its emergency checkpoint), this rank returns from ``fit()``
        normally. Needs a ``heartbeat`` coordinator (its store carries the note)."""
        if self.heartbeat is None:
            raise RuntimeError("leave_after_step needs Trainer(heartbeat=HeartbeatCoordinator(...))")
        self._leave_after = self.step + 1 if last_step is None else int(last_step)
        self.heartbeat.announce_departure(self._leave_after)

    def _check_peers_present(self) -> None:
        if self.heartbeat is None or not hasattr(self.heartbeat, "departed"):
            return
        gone = self.heartbeat.departed(self.step + 1)
        if gone:
            from ..fault_tolerance.hang_detection import PeerLeftError

            raise PeerLeftError(f"rank(s) {gone} left the job after step {self.step}: stopping before step "
                                f"{self.step + 1} is launched")

    # ------------------------------------------------------------------ loop
    def fit(self):
        if self.hang_detector is not None:
            self.hang_detector.start()
        if self.heartbeat is not None:
            self.heartbeat.start()
        for cb in self.callbacks:
            cb.pre_train(self)
        try:
            while self.step < self.config.max_steps and self._stop_reason is None:
                if self._leave_after is not None and self.step >= self._leave_after:
                    self._stop_reason = f"left the job after step {self.step}"
                    # this rank's state joins the peers' emergency checkpoints of the same step, so that a restart
                    # on the remaining ranks finds every shard
                    self.emergency_checkpoint_dir = self._emergency_checkpoint()
                    break
                self._check_peers_present()
                self._train_step_with_callbacks()
                if self.hang_detector is not None:
                    self.hang_detector.heartbeat()
                if self.heartbeat is not None:
                    self.heartbeat.heartbeat(self.step)
            if self._metrics and self._leave_after is None:   # a collective: not for a rank that leaves alone
                self._flush_metrics()
            for cb in self.callbacks:
                cb.post_train(self)
        except BaseException as e:  # noqa: BLE001
            for cb in self.callbacks:
                try:
                    cb.on_error(self, e)
                except Exception:  # noqa: BLE001
                    pass
            from ..fault_tolerance.hang_detection import CommTimeoutError

            if isinstance(e, CommTimeoutError):
                self.emergency_checkpoint_dir = self._emergency_checkpoint()
            raise
        finally:
            if self.hang_detector is not None:
                self.hang_detector.stop()
            if self.heartbeat is not None:
                self.heartbeat.stop()
            for cb in self.callbacks:
                cb.close(self)
        return self

    def _train_step_with_callbacks(self):
        c = self.config
        t0 = time.time()
        for cb in self.callbacks:
            cb.pre_load_batch(self)
        batches = [self._get_batch() for _ in range(c.gradient_accumulation_steps)]
        for cb in self.callbacks:
            cb.pre_step(self, batches[0])
        loss = self._train_step(batches)
        for cb in self.callbacks:
            cb.post_train_batch(self)
        grad_norm = None
        for cb in self.callbacks:
            cb.pre_optim_step(self)
        if self._arena_opt:
            self.optimizer.max_grad_norm = c.max_grad_norm
            self.optimizer.step()
            grad_norm = self.optimizer.last_grad_norm
        else:
            self._sync_replicated_grads()
            if c.max_grad_norm and c.max_grad_norm > 0:
                params = [p for p in self.model.parameters() if p.grad is not None]
                sharded = any(getattr(p, "_ep_sharded", False) or getattr(p, "_tp_sharded", None) is not None
                              for p in params) and dist.is_available() and dist.is_initialized()
                if getattr(self.model, "_pp_enabled", False) or sharded:
                    # one norm over every shard: tensor-parallel shards add up over their group, expert shards over the
                    # expert-parallel group, pipeline stages over the pipeline group
                    from ..parallel.pipeline_runtime import clip_grad_norm_pp

                    ep_group = next((m.ep.ep_group for m in self.model.modules()
                                     if hasattr(m, "ep") and getattr(m.ep, "ep_size", 1) > 1), None)
                    grad_norm = clip_grad_norm_pp(params, c.max_grad_norm, getattr(self.model, "_pp_group", None),
                                                  copies=2 if getattr(self.model, "is_dualpipe", False) else 1,
                                                  ep_group=ep_group)
                elif params and getattr(self.model, "_fsdp_extra_dims", None) is not None and dist.is_initialized() and (
                        self.model._fsdp_extra_dims.get("ep") is not None or getattr(self.model, "_tp_enabled", False)):
                    grad_norm = self._clip_fsdp_sharded(params, c.max_grad_norm)
                elif params:
                    grad_norm = torch.nn.utils.clip_grad_norm_(params, c.max_grad_norm)
            self.optimizer.step()
        if self.scheduler is not None:
            self.scheduler.step()
        self.optimizer.zero_grad(set_to_none=True)
        self._post_batch_hooks()
        self.step += 1
        self.tokens_seen += self.tokens_per_step
        self.record_metric("train/CE loss", loss)
        self.record_metric("train/PPL", torch.exp(loss.detach().float().clamp(max=20.0)) if torch.is_tensor(loss)
                           else math.exp(min(loss, 20.0)))
        if grad_norm is not None:
            self.record_metric("optim/total grad norm", grad_norm)
        self.record_metric("optim/LR", self.optimizer.param_groups[0]["lr"])
        self.record_metric("throughput/total tokens", self.tokens_seen)
        for cb in self.callbacks:
            cb.post_step(self)
        self.record_metric("throughput/step_time (s)", time.time() - t0)
        if c.log_interval and self.step % c.log_interval == 0:
            self._flush_metrics()
        if c.save_interval and self.step % c.save_interval == 0 and self.step > 0:
            self._save_checkpoint()

    def _grad_reducer(self):
        """Bucketed, backward-overlapped all-reduce over the ranks that hold the same parameters (``parallel/ddp.py``);
        built lazily for un-sharded data parallelism without the parameter arena."""
        if self._reducer is None and self.world_size > 1 and not getattr(self.model, "_fsdp_enabled", False) and \
                getattr(self.model, "_needs_grad_sync", False) and not self._arena_opt and self._compressor is None:
            from ..parallel.ddp import BucketedGradReducer

            group = getattr(self.model, "_replica_group", dist.group.WORLD)
            if group is not None:
                params = [p for p in self.model.parameters() if not getattr(p, "_ep_sharded", False)]
                self._reducer = BucketedGradReducer(params, group=group,
                                                    divisor=dist.get_world_size(group) / max(self.config.cp_size, 1))
        return self._reducer

    def _sync_replicated_grads(self):
        """Plain data parallelism for un-sharded models: finish the bucketed all-reduce started during backward, or,
        with gradient compression on, all-reduce the random projection of the flat gradient (error feedback keeps what
        the projection lost for the next step)."""
        if self._compressor is not None:
            if self.world_size > 1:
                ps = [p for p in self._compressed_params if p.grad is not None]
                if ps:
                    flat = torch.cat([p.grad.reshape(-1).float() for p in ps])
                    rec = self._compressor.all_reduce_gradients(flat)
                    off = 0
                    for p in ps:
                        n = p.numel()
                        p.grad.copy_(rec[off:off + n].view_as(p.grad))
                        off += n
            return
        r = self._grad_reducer()
        if r is not None:
            r.finish()
        self._sync_expert_replicas()
        self._sync_fsdp_extra_dims()

    def _clip_fsdp_sharded(self, params, max_norm: float):
        """Global-norm clipping of a PyTorch-FSDP2 model that also holds tensor-parallel or expert shards. FSDP2 replaces
        the parameter objects, so the shard marks are read off the modules: squared norms of the local gradient shards
        add up over the FSDP shard group; those of tensor-parallel weights also over the TP group and those of expert
        shards over the EP group, on whose ranks everything else is identical. (``clip_grad_norm_`` alone gives every
        rank a norm with only its own TP / expert shards in it, and the replicas drift apart.)"""
        from ..models.attention import Attention
        from ..models.feed_forward import FeedForward
        from ..models.moe import MoEBase

        expert_ids, tp_ids, tp_group = set(), set(), None
        for m in self.model.modules():
            if isinstance(m, MoEBase) and getattr(m.ep, "ep_size", 1) > 1:
                expert_ids |= {id(m.w1), id(m.w2), id(m.w3)}
            elif isinstance(m, (Attention, FeedForward)) and getattr(m, "_tp_size", 1) > 1:
                tp_group = m._tp_group
                for lin in ((m.w_q, m.w_k, m.w_v, m.w_out) if isinstance(m, Attention) else (m.w1, m.w3, m.w2)):
                    tp_ids.add(id(lin.weight))
                    if lin.bias is not None and lin not in (getattr(m, "w_out", None), getattr(m, "w2", None)):
                        tp_ids.add(id(lin.bias))      # column-parallel biases are shards; row-parallel ones are whole

        def local(g):
            return g._local_tensor if hasattr(g, "_local_tensor") else g

        t = torch.zeros(3, device=self.device, dtype=torch.float32)      # [whole, expert shards, TP shards]
        for p in params:
            k = 1 if id(p) in expert_ids else (2 if id(p) in tp_ids else 0)
            t[k] += local(p.grad).detach().float().pow(2).sum()
        shard_group = getattr(self.model, "_fsdp_shard_group", None)
        if shard_group is not None:
            dist.all_reduce(t, group=shard_group)
        ep_group = self.model._fsdp_extra_dims.get("ep")
        if ep_group is not None:
            dist.all_reduce(t[1:2], group=ep_group)
        if tp_group is not None:
            dist.all_reduce(t[2:], group=tp_group)
        total = t.sum().sqrt()
        coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
        for p in params:
            local(p.grad).mul_(coef.to(local(p.grad).dtype))
        return total

    def _sync_fsdp_extra_dims(self):
        """PyTorch FSDP2 reduce-scatters (averages) over the dp dims only. With expert parallelism the EP peers read
        other batches: gradients of everything but the expert shards are averaged over the EP group as well, and an
        expert shard's gradient - a sum over its EP sources, each scaled by its own rank's mean - is divided by the EP
        size so that every parameter ends up with the gradient of the mean over all ranks that read different batches.
        With context parallelism every gradient is a partial sum over the CP group and is summed there."""
        extra = getattr(self.model, "_fsdp_extra_dims", None)
        if not extra or not getattr(self.model, "_fsdp_enabled", False):
            return
        from ..models.moe import MoEBase

        expert_ids = set()
        for m in self.model.modules():
            if isinstance(m, MoEBase) and getattr(m.ep, "ep_size", 1) > 1:
                expert_ids |= {id(m.w1), id(m.w2), id(m.w3)}

        def local(g):
            return g._local_tensor if hasattr(g, "_local_tensor") else g

        ep_group, cp_group, sp_group = extra.get("ep"), extra.get("cp"), extra.get("sp")
        partial_ids = set()
        if sp_group is not None:     # whole parameters applied to row shards under sequence-parallel TP
            for m in self.model.modules():
                if isinstance(m, MoEBase):
                    partial_ids |= {id(q) for q in m.parameters()}
            for n, q in self.model.named_parameters():
                if "norm" in n or n.startswith("embeddings") or ".embeddings." in n:
                    partial_ids.add(id(q))
        for p in self.model.parameters():
            if p.grad is None:
                continue
            g = local(p.grad)
            if id(p) in partial_ids:
                dist.all_reduce(g, group=sp_group)
            if ep_group is not None:
                if id(p) not in expert_ids:
                    dist.all_reduce(g, group=ep_group)
                g.div_(dist.get_world_size(ep_group))
            if cp_group is not None:
                dist.all_reduce(g, group=cp_group)

    def _sync_expert_replicas(self):
        """Expert shards are left out of the replica reduction above (every expert-parallel rank holds other experts).
        An expert's gradient already collects the tokens of all expert-parallel peers, each with its own rank's
        mean-loss scale; what is missing is (1) the sum over the copies of the same shard on other data-parallel ranks
        (``ep_size`` below the data-parallel size) and (2) the division by the number of ranks that read different
        batches, which the replicated parameters get from their averaging all-reduce."""
        if not (dist.is_available() and dist.is_initialized()) or self._arena_opt:
            return
        ps = [p for p in self.model.parameters() if getattr(p, "_ep_sharded", False) and p.grad is not None]
        if not ps:
            return
        group = getattr(self.model, "_expert_replica_group", None)
        replica = getattr(self.model, "_replica_group", None)
        n_data = (dist.get_world_size(replica) if replica is not None else 1) / max(self.config.cp_size, 1)
        if group is not None and dist.get_world_size(group) > 1:
            flat = torch.cat([p.grad.reshape(-1).float() for p in ps])
            dist.all_reduce(flat, group=group)
            off = 0
            for p in ps:
                p.grad.copy_(flat[off:off + p.numel()].view_as(p.grad))
                off += p.numel()
        if n_data > 1:
            for p in ps:
                p.grad.div_(n_data)

    def _post_batch_hooks(self):
        """Per-step router updates (DeepSeek-V3 bias). A model that went through ``parallelize_model`` says which ranks
        hold the same layers and route other tokens (its replica group; under sequence-parallel TP also the TP group):
        the load counts are summed over exactly those. Any other model keeps the plain all-rank sum."""
        scoped = hasattr(self.model, "_replica_group") and dist.is_available() and dist.is_initialized()
        rep = getattr(self.model, "_replica_group", None)
        for m in self.model.modules():
            if hasattr(m, "post_batch") and hasattr(m, "score_bias"):
                if scoped:
                    m.post_batch(groups=[g for g in (rep, getattr(m, "_sp_group", None)) if g is not None])
                else:
                    m.post_batch()

    def _pipeline_step(self, batches):
        """One optimizer step of a pipeline stage: every batch runs through this rank's action list of the
        configured schedule (activations and gradients travel point to point); the loss is computed on the
        last stage and broadcast so that every rank logs the same value."""
        from ..parallel.pipeline_runtime import PipelineParallelConfig, PipelineSchedule, PipelineScheduleType

        c = self.config
        group = self.model._pp_group
        pp = dist.get_world_size(group)
        stages = list(self.model.stages) if hasattr(self.model, "stages") else [self.model]
        # context parallelism inside the stages: every CP rank runs the pipeline on its share of each sequence
        cp_group = getattr(stages[0], "_cp_group", None)
        cp = dist.get_world_size(cp_group) if cp_group is not None else 1
        if self._pp_schedule is None:
            m = c.pp_microbatches or pp
            assert c.micro_batch_size % m == 0, "micro_batch_size must be a multiple of the pipeline microbatch count"
            cfg = getattr(self.model, "_pp_config", None) or PipelineParallelConfig(
                degree=pp, schedule=PipelineScheduleType(c.pp_schedule), num_microbatches=m)
            assert cfg.stages_per_rank() == len(stages), \
                f"schedule {cfg.schedule} needs {cfg.stages_per_rank()} stage(s) per rank, the model holds {len(stages)}: " \
                "build it with parallelize_model(pp_config=...) or split_model() + PipelineStages"
            d_model = stages[0].d_model
            dtype = next(self.model.parameters()).dtype
            self._pp_schedule = PipelineSchedule(stages, group, cfg, num_microbatches=m,
                                                 hidden_shape=(c.micro_batch_size // m, c.sequence_length // cp, d_model),
                                                 hidden_dtype=dtype)
        self.model.train()
        total = torch.zeros((), device=self.device)
        reducer = self._grad_reducer()
        if reducer is not None:
            reducer.enabled = False   # many backward passes per step: the buckets go out once, in finish()
        for input_ids, labels in batches:
            input_ids = input_ids.to(self.device, non_blocking=True)
            labels = labels.to(self.device, non_blocking=True)
            kw = {}
            if cp > 1:
                from ..parallel.context_parallel import shard_batch_for_cp

                input_ids, labels = shard_batch_for_cp(input_ids, labels, cp, dist.get_rank(cp_group))
                kw["labels_shifted"] = True
            loss = self._pp_schedule.step(input_ids, target=labels, **kw)
            if loss is not None:
                total += loss.detach().float()
        total /= len(batches)
        if self._arena_opt:
            self.optimizer.grad_divisor = float(len(batches)) / cp     # CP ranks hold shares of one gradient: summed
        elif len(batches) > 1:
            for p in self.model.parameters():
                if p.grad is not None:
                    p.grad.div_(len(batches))
        if getattr(self.model, "is_dualpipe", False):
            from ..parallel.pipeline_runtime import sync_twin_grads, sync_twin_router_counts

            sync_twin_grads(stages, group, grad_of=(lambda q: getattr(q, "main_grad", None)) if self._arena_opt
                            else None)
            sync_twin_router_counts(stages, group)
        # every rank logs the loss of the last stage (rank p-1 for loop placements, rank 0 for the V placement, the mean
        # of ranks p-1 and 0 under DualPipe)
        return self._pp_schedule.loss_on_all_ranks(total)

    def _train_step(self, batches):
        if getattr(self.model, "_pp_enabled", False) and dist.is_initialized():
            return self._pipeline_step(batches)
        c = self.config
        accum = len(batches)
        total = None
        self.model.train()
        autocast_on = self.device.type == "cuda" and c.dtype in (torch.bfloat16, torch.float16) and \
            next(self.model.parameters()).dtype == torch.float32
        reducer = self._grad_reducer()
        arena = getattr(self.optimizer, "arena", None) if self._arena_opt else None
        if arena is not None:
            # read by the bucket reductions launched during backward. Context-parallel ranks each hold their share of one
            # sequence's gradient (the loss is already normalised by the global token count): those are summed, only
            # the data-parallel replicas are averaged
            self.optimizer.grad_divisor = float(accum) / max(self.config.cp_size, 1)
        for bi, (input_ids, labels) in enumerate(batches):
            if reducer is not None:
                reducer.enabled = bi == accum - 1   # gradients accumulate locally; reduce on the last micro-batch
            if arena is not None:
                arena.reduce_enabled = bi == accum - 1
            input_ids = input_ids.to(self.device, non_blocking=True)
            labels = labels.to(self.device, non_blocking=True)
            kw = {}
            cp_group = getattr(self.model, "_cp_group", None)
            if cp_group is not None:
                from ..parallel.context_parallel import shard_batch_for_cp

                input_ids, labels = shard_batch_for_cp(input_ids, labels, dist.get_world_size(cp_group),
                                                       dist.get_rank(cp_group))
                kw["labels_shifted"] = True
            with torch.autocast(device_type=self.device.type, dtype=c.dtype, enabled=autocast_on):
                out = self.model(input_ids, labels=labels, **kw)
            loss = out["loss"]
            aux = out.get("aux_loss") if isinstance(out, dict) else None
            full = loss if aux is None else loss + aux
            if not self._arena_opt:
                full = full / accum
            (full * c.loss_scale).backward()
            total = loss.detach() if total is None else total + loss.detach()
        return total / accum

    @staticmethod
    def _as_pair(batch):
        """``(input_ids, labels)`` from what a loader yields: a pair, or the reference's mapping with ``input_ids`` and
        ``labels`` (train/trainer.py:322-324; without ``labels`` the inputs are their own targets)."""
        if isinstance(batch, dict):
            ids = batch["input_ids"]
            labels = batch.get("labels")
            return ids, (ids if labels is None else labels)
        return batch

    def _get_batch(self):
        c = self.config
        if self.data_loader is not None:
            if self._data_iter is None:
                self._data_iter = iter(self.data_loader)
            try:
                return self._as_pair(next(self._data_iter))
            except StopIteration:
                if hasattr(self.data_loader, "set_epoch"):
                    self.data_loader.set_epoch(getattr(self.data_loader, "epoch", 0) + 1)
                self._data_iter = iter(self.data_loader)
                return self._as_pair(next(self._data_iter))
        ids = torch.randint(0, self.get_vocab_size(), (c.micro_batch_size, c.sequence_length))
        return ids, ids.clone()

    # ------------------------------------------------------------------ checkpoints
    def _save_checkpoint(self, is_best: bool = False):
        self.check_device_status("(before checkpoint)")
        if self.checkpointer is not None:
            self.checkpointer.save(self.step, self.model, self.optimizer, scheduler=self.scheduler,
                                   extra={"tokens_seen": self.tokens_seen, "best_val_loss": self._best_val_loss})
            return
        if not self.is_main:
            return
        os.makedirs(self.config.save_dir, exist_ok=True)
        state = {"step": self.step, "model_state_dict": self.model.state_dict(),
                 "optimizer_state_dict": self.optimizer.state_dict(), "best_val_loss": self._best_val_loss,
                 "scheduler_state_dict": self.scheduler.state_dict() if self.scheduler is not None else None}
        path = os.path.join(self.config.save_dir, f"step_{self.step:06d}.pt")
        torch.save(state, path)
        if is_best:
            torch.save(state, os.path.join(self.config.save_dir, "best.pt"))

    def load_checkpoint(self, path: str) -> int:
        if os.path.isdir(path) and self.checkpointer is not None:
            meta = self.checkpointer.load(path=path, model=self.model, optimizer=self.optimizer,
                                          scheduler=self.scheduler)
            self.step = int(meta.get("step", 0))
            self.tokens_seen = int((meta.get("extra") or {}).get("tokens_seen", 0))
            return self.step
        state = torch.load(path, map_location="cpu", weights_only=False)
        self.model.load_state_dict(state["model_state_dict"])
        self.optimizer.load_state_dict(state["optimizer_state_dict"])
        if self.scheduler is not None and state.get("scheduler_state_dict") is not None:
            self.scheduler.load_state_dict(state["scheduler_state_dict"])
        self.step = int(state.get("step", 0))
        self._best_val_loss = state.get("best_val_loss", float("inf"))
        return self.step
