"""Pipeline schedule generators: GPipe, 1F1B, Zero-Bubble and DualPipe
(reference: distributed/pipeline_parallel.py:44-472).

Every generator returns per-rank action lists and every list is checked by ``validate_schedule``,
a dependency simulator (F needs the previous stage's F, B needs this stage's F and the next stage's
B, W needs this stage's B). The simulator also measures the bubble, so the closed-form
``compute_bubble_fraction`` can be compared with what a schedule really does. The reference's
DualPipe generator emits duplicate forwards and its Zero-Bubble has no separate weight-gradient
action; here B (input gradient) and W (weight gradient) are distinct action types and DualPipe is a
true two-direction schedule (rank r runs stage r of direction 0 and stage p-1-r of direction 1).
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


class ScheduleType(Enum):
    # FWD / BWD / IDLE with the reference's values (distributed/pipeline_parallel.py: auto() = 1, 2, 3)
    FWD = 1
    BWD = 2              # full backward (input + weight gradients)
    IDLE = 3
    BWD_INPUT = 4        # zero-bubble "B": input gradients only
    BWD_WEIGHT = 5       # zero-bubble "W": weight gradients only


@dataclass(frozen=True)
class Action:
    type: ScheduleType
    microbatch: int = -1
    stage: int = -1

    # the reference's field names (distributed/pipeline_parallel.py:62-68)
    @property
    def microbatch_idx(self) -> int:
        return self.microbatch

    @property
    def stage_idx(self) -> int:
        return self.stage

    def __repr__(self):
        tag = {ScheduleType.FWD: "F", ScheduleType.BWD: "B", ScheduleType.BWD_INPUT: "Bi", ScheduleType.BWD_WEIGHT: "W",
               ScheduleType.IDLE: "-"}[self.type]
        return f"{tag}{self.microbatch}@{self.stage}" if self.type != ScheduleType.IDLE else "-"


@dataclass
class PipelineParallelConfig:
    degree: int = 1
    schedule: str = "1f1b"
    num_microbatches: Optional[int] = None


class PipelineStage(nn.Module):
    """A contiguous slice of layers with p2p helpers (reference: distributed/pipeline_parallel.py:71-149).
    Sends/receives are non-blocking ``batch_isend_irecv`` pairs on the PP group."""

    def __init__(self, layers=None, stage_id=None, num_stages: Optional[int] = None, group=None, *,
                 stage_idx: Optional[int] = None, loss_fn=None):
        """``PipelineStage(layers, stage_id, num_stages)``; the reference's ``PipelineStage(stage_idx, num_stages, layers,
        loss_fn)`` (distributed/pipeline_parallel.py) is recognised by its first argument being an int."""
        super().__init__()
        if isinstance(layers, int) and not isinstance(layers, bool):      # reference order: (stage_idx, num_stages, layers)
            layers, stage_id, num_stages = num_stages, layers, stage_id
        if stage_idx is not None:
            stage_id = stage_idx
        self.layers = layers
        self.stage_id, self.num_stages, self.group = stage_id, num_stages, group
        self.loss_fn = loss_fn

    @property
    def is_first(self) -> bool:
        return self.stage_id == 0

    @property
    def is_last(self) -> bool:
        return self.stage_id == self.num_stages - 1

    def forward_chunk(self, x, labels=None, is_last_chunk: bool = False, **kw):
        """The stage's layers on ``x``; on the last chunk, with ``labels`` and a ``loss_fn`` (the head), also the
        cross-entropy of ``loss_fn(x)``: ``(x, loss)`` (reference: distributed/pipeline_parallel.py:101-129)."""
        if isinstance(self.layers, (nn.ModuleList, nn.Sequential)):
            for l in self.layers:
                x = l(x, **kw) if kw else l(x)
        else:
            x = self.layers(x, **kw)
        if is_last_chunk and self.loss_fn is not None and labels is not None:
            logits = self.loss_fn(x)
            loss = torch.nn.functional.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), labels.reshape(-1),
                                                     ignore_index=-100)
            return x, loss
        return x

    forward = forward_chunk

    def _peer(self, delta: int) -> int:
        r = dist.get_rank(self.group)
        n = dist.get_world_size(self.group)
        return dist.get_global_rank(self.group, (r + delta) % n) if self.group is not None else (r + delta) % n

    def send_forward(self, x):
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, x.contiguous(), self._peer(+1), group=self.group)])

    def recv_forward(self, x):
        """``x``: the buffer to receive into."""
        return dist.batch_isend_irecv([dist.P2POp(dist.irecv, x, self._peer(-1), group=self.group)])

    def send_backward(self, grad):
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, grad.contiguous(), self._peer(-1), group=self.group)])

    def recv_backward(self, grad):
        """``grad``: the buffer to receive into."""
        return dist.batch_isend_irecv([dist.P2POp(dist.irecv, grad, self._peer(+1), group=self.group)])


# ------------------------------------------------------------------ generators
F, B, BI, W = ScheduleType.FWD, ScheduleType.BWD, ScheduleType.BWD_INPUT, ScheduleType.BWD_WEIGHT


class PerRankSchedule(list):
    """What every generator returns: ``schedule[rank]`` is that rank's action list. Also reads like the mapping that
    the reference's DualPipe generator returns (``for rank, actions in schedule.items()``;
    distributed/pipeline_parallel.py), so code written against either shape keeps working."""

    def keys(self):
        return range(len(self))

    def values(self):
        return list(self)

    def items(self):
        return list(enumerate(self))

    def get(self, rank, default=None):
        return self[rank] if isinstance(rank, int) and 0 <= rank < len(self) else default


class _Schedule:
    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        fn = cls.__dict__.get("generate_schedule")
        if fn is not None:
            def generate_schedule(self, *a, _fn=fn, **k):
                out = _fn(self, *a, **k)
                return out if isinstance(out, PerRankSchedule) else PerRankSchedule(out)

            generate_schedule.__doc__ = fn.__doc__
            cls.generate_schedule = generate_schedule

    def __init__(self, num_stages=None, num_microbatches: int = 1, *, stages=None):
        """``num_stages``: the pipeline depth, or - the reference's form, ``GPipeSchedule(stages, num_microbatches)``
        (distributed/pipeline_parallel.py) - the list of stage modules, of which only the length matters here."""
        if stages is not None and num_stages is None:
            num_stages = stages
        if not isinstance(num_stages, int):
            self.stages = list(num_stages)
            num_stages = len(self.stages)
        self.num_stages = num_stages
        self.num_microbatches = num_microbatches

    def generate_schedule(self) -> List[List[Action]]:
        raise NotImplementedError

    def rank_of_stage(self, stage: int) -> int:
        return stage

    def stages_of_rank(self, rank: int) -> List[int]:
        return [rank]


class GPipeSchedule(_Schedule):
    def generate_schedule(self):
        p, m = self.num_stages, self.num_microbatches
        return [[Action(F, i, r) for i in range(m)] + [Action(B, i, r) for i in reversed(range(m))]
                for r in range(p)]


class OneForwardOneBackwardSchedule(_Schedule):
    def generate_schedule(self):
        p, m = self.num_stages, self.num_microbatches
        out = []
        for r in range(p):
            warm = min(p - 1 - r, m)
            acts = [Action(F, i, r) for i in range(warm)]
            f, b = warm, 0
            while b < m:
                if f < m:
                    acts.append(Action(F, f, r))
                    f += 1
                acts.append(Action(B, b, r))
                b += 1
            out.append(acts)
        return out


def _greedy(p: int, work: Dict[int, List[List[Action]]], stage_rank, last_stage_of, first_stage_of,
                  split_w: bool, costs=None) -> List[List[Action]]:
    """List scheduling shared by the interleaved, Zero-Bubble and DualPipe generators: every rank holds one ordered
    queue of F and B actions per stage (or direction). It works with durations, not ticks: an unsplit backward costs
    twice a forward, so a rank that has just finished a forward may find the gradient it waits for still one forward
    away and should run another forward meanwhile, which a scheduler that advances every rank by one action per tick
    cannot see (interleaved 1F1B at p = 4, m = 8: 18.6 % idle instead of 28.4 %). At each step the
    action that can start earliest on any rank is placed (a ready backward before a ready forward, alternating between
    a rank's queues); a rank with nothing startable at its clock runs a pending W if it has one, else idles until its
    earliest head becomes ready."""
    costs = costs or {F: 1.0, B: 2.0, BI: 1.0, W: 1.0}
    finish: Dict[tuple, float] = {}
    clock = [0.0] * p
    pending_w: List[List[Action]] = [[] for _ in range(p)]
    out: List[List[Action]] = [[] for _ in range(p)]
    queues = {r: [list(q) for q in work[r]] for r in range(p)}
    turn = [0] * p
    INF = float("inf")

    def ready_time(a: Action) -> float:
        """Earliest start allowed by the dependencies that are already placed; ``INF`` while one is not."""
        deps = []
        if a.type == F:
            if a.stage != first_stage_of(a):
                deps.append(("F", a.microbatch, a.stage - 1))
        else:
            deps.append(("F", a.microbatch, a.stage))
            if a.stage != last_stage_of(a):
                deps.append(("B", a.microbatch, a.stage + 1))
        t = 0.0
        for d in deps:
            if d not in finish:
                return INF
            t = max(t, finish[d])
        return t

    total = sum(len(q) for r in range(p) for q in queues[r])
    guard = 0
    while total > 0:
        guard += 1
        if guard > 1000000:
            raise RuntimeError("schedule generation did not converge")
        best = None   # (start, is_forward, queue distance, rank, queue index)
        for r in range(p):
            for qi, q in enumerate(queues[r]):
                if not q:
                    continue
                rt = ready_time(q[0])
                if rt == INF:
                    continue
                start = max(rt, clock[r])
                key = (start, 1 if q[0].type == F else 0, (qi - turn[r]) % max(len(queues[r]), 1), r, qi)
                if best is None or key < best:
                    best = key
        if best is None:
            raise RuntimeError("no action can start: the queues do not form a valid pipeline")
        start, _, _, r, qi = best
        # fill the wait before `start` with deferred weight-gradient work (it needs nothing from other ranks)
        while pending_w[r] and clock[r] + costs[W] <= start + 1e-9:
            out[r].append(pending_w[r].pop(0))
            clock[r] += costs[W]
        start = max(start, clock[r])
        a = queues[r][qi].pop(0)
        turn[r] = (qi + 1) % len(queues[r])
        if a.type == F:
            out[r].append(a)
            dur, tag = costs[F], "F"
        else:
            out[r].append(Action(BI if split_w else B, a.microbatch, a.stage))
            dur, tag = (costs[BI] if split_w else costs[B]), "B"
            if split_w:
                pending_w[r].append(Action(W, a.microbatch, a.stage))
        clock[r] = start + dur
        finish[(tag, a.microbatch, a.stage)] = clock[r]
        total -= 1
    for r in range(p):
        out[r] += pending_w[r]
    return out


def _one_f_one_b_queue(stage: int, pos: int, depth: int, mbs: List[int]) -> List[Action]:
    """1F1B order of one stage that sits at position ``pos`` of a ``depth``-stage pipeline."""
    warm = min(depth - 1 - pos, len(mbs))
    acts = [Action(F, mb, stage) for mb in mbs[:warm]]
    f, b = warm, 0
    while b < len(mbs):
        if f < len(mbs):
            acts.append(Action(F, mbs[f], stage))
            f += 1
        acts.append(Action(B, mbs[b], stage))
        b += 1
    return acts


class InterleavedSchedule(_Schedule):
    """``v`` model chunks per rank. ``placement="loop"``: stage s lives on rank ``s % p`` (interleaved
    1F1B / looped BFS); ``"v"``: the second half of the stages runs back down the ranks (ZB-V). With
    ``split_w`` the backward is split into B and W and W fills idle slots."""

    def __init__(self, num_ranks: int, num_microbatches: int, v: int = 2, placement: str = "loop",
                 split_w: bool = False, order: str = "1f1b"):
        """``order="bfs"``: looped breadth-first - every stage runs all its forwards before any backward (the GPipe
        order per model chunk), which keeps the most activations alive and the fewest transfers in flight."""
        super().__init__(num_ranks, num_microbatches)
        self.v, self.placement, self.split_w, self.order = v, placement, split_w, order
        self.total_stages = v * num_ranks

    def rank_of_stage(self, stage: int) -> int:
        p = self.num_stages
        if self.placement == "v":
            c, r = divmod(stage, p)
            return r if c % 2 == 0 else p - 1 - r
        return stage % p

    def stages_of_rank(self, rank: int) -> List[int]:
        return [s for s in range(self.total_stages) if self.rank_of_stage(s) == rank]

    def generate_schedule(self):
        p, m, S = self.num_stages, self.num_microbatches, self.total_stages
        mbs = list(range(m))
        if self.order == "bfs":
            work = {r: [[Action(F, mb, s) for mb in mbs] + [Action(B, mb, s) for mb in mbs]
                        for s in self.stages_of_rank(r)] for r in range(p)}
        elif self.order == "1f1b" and self.placement == "loop" and not self.split_w and m % p == 0:
            # The depth-first interleaved order (Narayanan et al. 2021): micro-batches advance in groups of p through
            # chunk 0, chunk 1, ...; rank r warms up with 2 (p - r - 1) + (v - 1) p forwards, then alternates one
            # forward and one backward. One fixed queue per rank; the list scheduler only checks that it is feasible.
            v, total = self.v, m * self.v

            def fwd(k, r):
                return Action(F, (k // (p * v)) * p + k % p, ((k // p) % v) * p + r)

            def bwd(k, r):
                return Action(B, (k // (p * v)) * p + k % p, (v - 1 - (k // p) % v) * p + r)

            work = {}
            for r in range(p):
                warm = min(2 * (p - r - 1) + (v - 1) * p, total)
                q = [fwd(k, r) for k in range(warm)]
                for i in range(total - warm):
                    q += [fwd(warm + i, r), bwd(i, r)]
                q += [bwd(i, r) for i in range(total - warm, total)]
                work[r] = [q]
        else:
            work = {r: [_one_f_one_b_queue(s, s, S, mbs) for s in self.stages_of_rank(r)] for r in range(p)}
        return _greedy(p, work, self.rank_of_stage, lambda a: S - 1, lambda a: 0, split_w=self.split_w)


class ZeroBubbleSchedule(_Schedule):
    """ZB-H1 style: 1F1B order with the backward split into B and W; W fills what would be bubbles."""

    def generate_schedule(self):
        p, m = self.num_stages, self.num_microbatches
        base = OneForwardOneBackwardSchedule(p, m).generate_schedule()
        work = {r: [base[r]] for r in range(p)}
        return _greedy(p, work, lambda s: s, lambda a: p - 1, lambda a: 0, split_w=True)


class DualPipeSchedule(_Schedule):
    """Two pipelines in opposite directions over the same ranks. Stage ids ``0..p-1`` are direction
    0 (stage s on rank s), ``p..2p-1`` direction 1 (stage p+s on rank p-1-s); even microbatches go
    down direction 0, odd ones direction 1. ``stages_forward`` / ``stages_reverse`` are accepted for
    signature parity with the reference and only their length is used."""

    def __init__(self, stages_forward=None, stages_reverse=None, num_microbatches: int = 8,
                 num_stages: Optional[int] = None, split_w: bool = True):
        p = num_stages or (len(stages_forward) if stages_forward is not None else 2)
        super().__init__(p, num_microbatches)
        self.split_w = split_w

    def rank_of_stage(self, stage: int) -> int:
        p = self.num_stages
        return stage if stage < p else p - 1 - (stage - p)

    def stages_of_rank(self, rank: int) -> List[int]:
        p = self.num_stages
        return [rank, p + (p - 1 - rank)]

    def generate_schedule(self):
        p, m = self.num_stages, self.num_microbatches
        work: Dict[int, List[List[Action]]] = {}
        for r in range(p):
            qs = []
            for d in (0, 1):
                mbs = [i for i in range(m) if i % 2 == d]
                stage = r if d == 0 else p + (p - 1 - r)
                pos = stage - d * p
                warm = min(p - 1 - pos, len(mbs))
                acts = [Action(F, mb, stage) for mb in mbs[:warm]]
                f, b = warm, 0
                while b < len(mbs):
                    if f < len(mbs):
                        acts.append(Action(F, mbs[f], stage))
                        f += 1
                    acts.append(Action(B, mbs[b], stage))
                    b += 1
                qs.append(acts)
            work[r] = qs
        last = lambda a: (p - 1) if a.stage < p else (2 * p - 1)  # noqa: E731
        first = lambda a: 0 if a.stage < p else p  # noqa: E731
        return _greedy(p, work, self.rank_of_stage, last, first, split_w=self.split_w)


# ------------------------------------------------------------------ validation / bubble
def validate_schedule(per_rank: List[List[Action]], num_stages: int, num_microbatches: int,
                      stage_first=None, stage_last=None, mb_stages=None, costs=None) -> dict:
    """Simulate the schedule; raises ``ValueError`` on a missing/duplicate action or a deadlock.
    Returns ``{"makespan", "busy", "bubble_fraction"}`` with unit (or given) costs per action type."""
    costs = costs or {F: 1.0, B: 2.0, BI: 1.0, W: 1.0}
    stage_first = stage_first or (lambda s: 0)
    stage_last = stage_last or (lambda s: num_stages - 1)
    seen = set()
    for r, acts in enumerate(per_rank):
        for a in acts:
            if a.type == ScheduleType.IDLE:
                continue
            key = (a.type, a.microbatch, a.stage)
            if key in seen:
                raise ValueError(f"duplicate action {a} on rank {r}")
            seen.add(key)
    finish: Dict[tuple, float] = {}
    ptr = [0] * len(per_rank)
    clock = [0.0] * len(per_rank)
    busy = [0.0] * len(per_rank)
    remaining = sum(1 for acts in per_rank for a in acts if a.type != ScheduleType.IDLE)
    while remaining:
        progressed = False
        for r, acts in enumerate(per_rank):
            while ptr[r] < len(acts) and acts[ptr[r]].type == ScheduleType.IDLE:
                ptr[r] += 1
            if ptr[r] >= len(acts):
                continue
            a = acts[ptr[r]]
            deps = []
            if a.type == F:
                if a.stage != stage_first(a.stage):
                    deps.append(("F", a.microbatch, a.stage - 1))
            elif a.type in (B, BI):
                deps.append(("F", a.microbatch, a.stage))
                if a.stage != stage_last(a.stage):
                    deps.append(("B", a.microbatch, a.stage + 1))
            else:
                deps.append(("B", a.microbatch, a.stage))
            if all(d in finish for d in deps):
                start = max([clock[r]] + [finish[d] for d in deps])
                end = start + costs[a.type]
                kind = "F" if a.type == F else ("W" if a.type == W else "B")
                finish[(kind, a.microbatch, a.stage)] = end
                clock[r] = end
                busy[r] += costs[a.type]
                ptr[r] += 1
                remaining -= 1
                progressed = True
        if not progressed:
            raise ValueError("schedule deadlocks: no rank can make progress")
    makespan = max(clock)
    return {"makespan": makespan, "busy": busy,
            "bubble_fraction": 1.0 - sum(busy) / (makespan * len(per_rank)) if makespan > 0 else 0.0}


def compute_bubble_fraction(schedule_type: str, p: int, m: int, v: int = 1) -> float:
    """Closed-form bubble fractions (reference: distributed/pipeline_parallel.py:449-472)."""
    s = str(getattr(schedule_type, "value", schedule_type)).lower()
    if s in ("gpipe", "1f1b", "onef_oneb"):
        return (p - 1) / m
    if s in ("interleaved", "interleaved1f1b", "interleaved_1f1b", "loopedbfs", "looped_bfs"):
        return (p - 1) / (v * m)
    if s in ("dualpipe", "dual_pipe"):
        return max(p // 2 - 1, 0) / m
    if s in ("zb1p", "zero_bubble", "zerobubble", "zb-1p", "interleavedzerobubble"):
        return (p - 1) / (3 * (m + p - 1))
    if s in ("zb2p", "zbv", "zb-v", "zbvzerobubble", "zb-2p"):
        return 0.0
    raise ValueError(f"unknown schedule type {schedule_type}")
