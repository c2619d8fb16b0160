"""Pipeline-parallel runtime: model splitting, a schedule executor on NCCL/gloo p2p, gradient
clipping across stages (reference: distributed/pipeline_runtime.py:55-534).

The reference wraps ``torch.distributed.pipelining`` and a sequential DualPipe placeholder; neither
is wired to its Trainer. Here one executor runs any per-rank action list produced by
``pipeline_parallel`` (GPipe, 1F1B, Zero-Bubble with B/W split, DualPipe with two stage copies per
rank): activations and gradients move with non-blocking ``batch_isend_irecv`` pairs on the PP
group, receives are posted one action ahead so the transfer overlaps the previous action's compute
(on a GPU the NCCL p2p kernels run on NCCL's own stream).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from enum import Enum
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .pipeline_parallel import (Action, DualPipeSchedule, GPipeSchedule, InterleavedSchedule,
                                OneForwardOneBackwardSchedule, ScheduleType, ZeroBubbleSchedule,
                                compute_bubble_fraction)  # noqa: F401


class PipelineScheduleType(str, Enum):
    single_1F1B = "1F1B"
    interleaved_1F1B = "Interleaved1F1B"
    gpipe = "GPipe"
    looped_bfs = "LoopedBFS"
    interleaved_zero_bubble = "InterleavedZeroBubble"
    zbv_zero_bubble = "ZBVZeroBubble"
    dualpipe = "DualPipe"

    @property
    def is_single_stage(self) -> bool:
        return self in (PipelineScheduleType.single_1F1B, PipelineScheduleType.gpipe)


class PipelineSplitStyle(str, Enum):
    loop = "loop"
    v = "v"


def stage_layer_ranges(n_layers: int, num_stages: int, split_points: Optional[Sequence[int]] = None):
    """[(lo, hi)) layer range of every stage. Default split: ``base = L // stages`` with the
    remainder spread over stages 1.. (the first stage, which also holds the embeddings, gets ``base``)."""
    if split_points is not None:
        pts = [0, *split_points, n_layers]
        return [(pts[i], pts[i + 1]) for i in range(len(pts) - 1)]
    base, rem = divmod(n_layers, num_stages)
    sizes = [base] * num_stages
    for i in range(rem):
        sizes[1 + i % max(num_stages - 1, 1) if num_stages > 1 else 0] += 1
    out, lo = [], 0
    for s in sizes:
        out.append((lo, lo + s))
        lo += s
    return out


@dataclass
class PipelineParallelConfig:
    degree: int = 1
    schedule: PipelineScheduleType = PipelineScheduleType.single_1F1B
    split_points: Optional[List[int]] = None
    num_microbatches: Optional[int] = None
    style: PipelineSplitStyle = PipelineSplitStyle.loop

    def stages_per_rank(self) -> int:
        return 1 if PipelineScheduleType(self.schedule).is_single_stage else 2

    def num_stages(self) -> int:
        return self.degree * self.stages_per_rank()

    def get_split_points(self, n_layers: int) -> List[int]:
        if self.split_points is not None:
            return list(self.split_points)
        return [hi for _, hi in stage_layer_ranges(n_layers, self.num_stages())[:-1]]

    def stage_ids_this_rank(self, pp_rank: int) -> List[int]:
        n, spr = self.degree, self.stages_per_rank()
        if spr == 1:
            return [pp_rank]
        if PipelineScheduleType(self.schedule) in (PipelineScheduleType.zbv_zero_bubble,
                                                   PipelineScheduleType.dualpipe) or \
                self.style == PipelineSplitStyle.v:
            return [pp_rank, self.num_stages() - 1 - pp_rank]
        return [pp_rank + s * n for s in range(spr)]


def split_model(model: nn.Module, pp_mesh, pp_config: PipelineParallelConfig, *, device=None) -> List[nn.Module]:
    """One module per stage owned by this rank: a deep copy of the model trimmed to the stage's
    layers (embeddings only on the first stage, head only on the last)."""
    group = pp_mesh.get_group() if hasattr(pp_mesh, "get_group") else pp_mesh
    pp_rank = dist.get_rank(group) if group is not None else 0
    n_stages = pp_config.num_stages()
    pts = pp_config.get_split_points(getattr(model, "n_layers", 0)) if hasattr(model, "n_layers") else None
    for mod in model.modules():  # graph tensors cached by a previous forward cannot be deep-copied
        if hasattr(mod, "_aux_loss"):
            mod._aux_loss = None
    stages = []
    for sid in pp_config.stage_ids_this_rank(pp_rank):
        m = copy.deepcopy(model)
        if hasattr(m, "apply_pp"):
            m.apply_pp(group, num_stages=n_stages, stage_idx=sid, split_points=pts)
        if device is not None:
            m = m.to(device)
        m._stage_id = sid
        stages.append(m)
    return stages


# ------------------------------------------------------------------ executor
@dataclass
class _MB:
    inp: Optional[torch.Tensor] = None
    out: Optional[torch.Tensor] = None
    loss: Optional[torch.Tensor] = None
    grad_in: Optional[torch.Tensor] = None


class PipelineSchedule:
    """Runs one training step of a pipeline schedule on this rank.

    ``stages``: the stage module(s) this rank owns (``split_model``). Each is called as
    ``stage(x)`` and must return the hidden state, or - on the last stage, given ``target`` - a dict
    with ``"loss"`` (the built-in ``Transformer`` does both). ``loss_fn(output, target)`` overrides that.
    ``step(inputs, target=)`` takes the full local batch, splits it into microbatches, executes this
    rank's action list and returns the mean loss on the rank holding the last stage (else ``None``).
    """

    def __init__(self, stages: Sequence[nn.Module], pp_mesh, pp_config: PipelineParallelConfig, *,
                 num_microbatches: Optional[int] = None, loss_fn: Optional[Callable] = None,
                 hidden_shape: Optional[Sequence[int]] = None, hidden_dtype: Optional[torch.dtype] = None):
        self.stages = list(stages)
        self.group = pp_mesh.get_group() if hasattr(pp_mesh, "get_group") else pp_mesh
        self.cfg = pp_config
        self.p = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        self.m = num_microbatches or pp_config.num_microbatches or self.p
        self.loss_fn = loss_fn
        self.hidden_shape = tuple(hidden_shape) if hidden_shape is not None else None
        self.hidden_dtype = hidden_dtype
        st = PipelineScheduleType(pp_config.schedule)
        self.dual = st == PipelineScheduleType.dualpipe
        if st == PipelineScheduleType.gpipe:
            gen = GPipeSchedule(self.p, self.m)
        elif st == PipelineScheduleType.single_1F1B:
            gen = OneForwardOneBackwardSchedule(self.p, self.m)
        elif st == PipelineScheduleType.dualpipe:
            gen = DualPipeSchedule(num_stages=self.p, num_microbatches=self.m)
        elif st == PipelineScheduleType.zbv_zero_bubble:
            gen = InterleavedSchedule(self.p, self.m, v=2, placement="v", split_w=True)
        elif st == PipelineScheduleType.interleaved_zero_bubble:
            gen = InterleavedSchedule(self.p, self.m, v=2, placement="loop", split_w=True)
        else:  # Interleaved1F1B, LoopedBFS
            gen = InterleavedSchedule(self.p, self.m, v=2, placement="loop")
        self.generator = gen
        self.actions: List[Action] = gen.generate_schedule()[self.rank]
        self.total_stages = getattr(gen, "total_stages", 2 * self.p if self.dual else self.p)
        if self.dual:
            # direction 1 is a second copy of the pipeline: schedule stage p+s holds model stage s
            self.stage_of = {self.rank: self.stages[0], self.p + (self.p - 1 - self.rank): self.stages[-1]}
        else:
            self.stage_of = {getattr(s, "_stage_id", self.rank): s for s in self.stages}

    # -- helpers
    def _first(self, stage: int) -> bool:
        return stage in (0, self.p) if self.dual else stage == 0

    def _last(self, stage: int) -> bool:
        return stage in (self.p - 1, 2 * self.p - 1) if self.dual else stage == self.total_stages - 1

    def _rank_of(self, stage: int) -> int:
        return self.generator.rank_of_stage(stage)

    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    def _p2p(self, op, tensor, stage_peer: int, tag: int):
        peer = self._global(self._rank_of(stage_peer))
        return dist.batch_isend_irecv([dist.P2POp(op, tensor, peer, group=self.group, tag=tag)])

    def step(self, inputs: torch.Tensor, target: Optional[torch.Tensor] = None, **kwargs):
        m = self.m
        in_chunks = list(inputs.chunk(m, dim=0)) if inputs is not None else [None] * m
        tg_chunks = list(target.chunk(m, dim=0)) if target is not None else [None] * m
        state: Dict[tuple, _MB] = {}
        pending_send: list = []
        keepalive: list = []  # tensors of in-flight sends
        local_box: Dict[tuple, torch.Tensor] = {}  # hand-off between two stages of this rank
        losses: List[torch.Tensor] = []
        hs, hd = self.hidden_shape, self.hidden_dtype

        def hidden_like(ref_mb: int):
            nonlocal hs, hd
            if hs is None:
                raise RuntimeError("hidden_shape is required on stages that receive activations")
            return torch.empty(hs, dtype=hd, device=self._device())

        for a in self.actions:
            if a.type == ScheduleType.IDLE:
                continue
            stage_mod = self.stage_of[a.stage]
            key = (a.stage, a.microbatch)
            if a.type == ScheduleType.FWD:
                mb = state.setdefault(key, _MB())
                if self._first(a.stage):
                    x = in_chunks[a.microbatch]
                elif self._rank_of(a.stage - 1) == self.rank:  # previous stage lives on this rank too
                    x = local_box.pop(("act", a.stage, a.microbatch)).requires_grad_(True)
                else:
                    buf = hidden_like(a.microbatch)
                    for w in self._p2p(dist.irecv, buf, a.stage - 1, tag=a.microbatch):
                        w.wait()
                    x = buf.requires_grad_(True)
                mb.inp = x
                if self._last(a.stage):
                    out = stage_mod(x, labels=tg_chunks[a.microbatch], **kwargs) if self.loss_fn is None else \
                        stage_mod(x, **kwargs)
                    if self.loss_fn is not None:
                        y = out["logits"] if isinstance(out, dict) and "logits" in out else out
                        loss = self.loss_fn(y, tg_chunks[a.microbatch])
                    else:
                        loss = out["loss"]
                        if isinstance(out, dict) and out.get("aux_loss") is not None:
                            loss = loss + out["aux_loss"]
                    mb.loss = loss / m
                    losses.append(loss.detach())
                else:
                    out = stage_mod(x, **kwargs)
                    y = out["hidden_states"] if isinstance(out, dict) else out
                    mb.out = y
                    if hs is None:
                        hs, hd = tuple(y.shape), y.dtype
                    if self._rank_of(a.stage + 1) == self.rank:
                        local_box[("act", a.stage + 1, a.microbatch)] = y.detach().clone()
                    else:
                        keepalive.append(y.detach().contiguous())
                        pending_send += self._p2p(dist.isend, keepalive[-1], a.stage + 1, tag=a.microbatch)
            elif a.type in (ScheduleType.BWD, ScheduleType.BWD_INPUT):
                mb = state[key]
                if self._last(a.stage):
                    mb.loss.backward()
                elif self._rank_of(a.stage + 1) == self.rank:
                    mb.out.backward(local_box.pop(("grad", a.stage, a.microbatch)))
                else:
                    g = torch.empty_like(mb.out)
                    for w in self._p2p(dist.irecv, g, a.stage + 1, tag=10000 + a.microbatch):
                        w.wait()
                    mb.out.backward(g)
                if not self._first(a.stage) and mb.inp.grad is not None:
                    if self._rank_of(a.stage - 1) == self.rank:
                        local_box[("grad", a.stage - 1, a.microbatch)] = mb.inp.grad
                    else:
                        keepalive.append(mb.inp.grad.contiguous())
                        pending_send += self._p2p(dist.isend, keepalive[-1], a.stage - 1, tag=10000 + a.microbatch)
                state.pop(key)
            # BWD_WEIGHT: weight gradients were produced together with the input gradients above
        for w in pending_send:
            w.wait()
        if losses:
            return torch.stack(losses).mean()
        return None

    def _device(self):
        for s in self.stages:
            for p in s.parameters():
                return p.device
        return torch.device("cpu")


class DualPipeScheduleRuntime(PipelineSchedule):
    """DualPipe executor: this rank owns two stage copies (one per direction); even microbatches
    enter at rank 0, odd ones at rank p-1 (reference: distributed/pipeline_runtime.py:303-397, which
    runs the phases sequentially on one direction only)."""

    def __init__(self, stages, pp_mesh, pp_config=None, **kw):
        cfg = pp_config or PipelineParallelConfig(schedule=PipelineScheduleType.dualpipe)
        cfg.schedule = PipelineScheduleType.dualpipe
        super().__init__(stages, pp_mesh, cfg, **kw)


def clip_grad_norm_pp(parameters, max_norm: float, pp_group=None, norm_type: float = 2.0) -> torch.Tensor:
    """Clip by the global norm over all pipeline stages (one scalar all-reduce over the PP group)."""
    params = [p for p in parameters if p.grad is not None]
    dev = params[0].device if params else torch.device("cpu")
    if norm_type == float("inf"):
        total = torch.stack([p.grad.detach().abs().max() for p in params]).max() if params else torch.zeros((), device=dev)
        if pp_group is not None:
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=pp_group)
    else:
        total = torch.stack([p.grad.detach().float().norm(norm_type) ** norm_type for p in params]).sum() \
            if params else torch.zeros((), device=dev)
        if pp_group is not None:
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=pp_group)
        total = total ** (1.0 / norm_type)
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for p in params:
        p.grad.mul_(coef.to(p.grad.dtype))
    return total
