"""Replays the pipeline executor's point-to-point traffic under NCCL's ordering rules, on the host.

gloo delivers point-to-point messages independently of one another, so a CPU test of a schedule cannot see the two
ways the same program can stand still on NCCL:

* every operation of one communicator runs on one stream per rank, in the order it was issued, and a send (receive)
  completes only once the matching receive (send) has reached the head of *its* stream: a receive posted early blocks
  whatever this rank issues on the same communicator afterwards until the peer sends;
* messages between a pair on one communicator match by order, not by tag.

``trace_rank`` runs the real ``PipelineSchedule.step`` of one rank with dummy stages against a transport that records
(post receive, wait, send, compute) instead of communicating; the host of the real executor never blocks on the device,
so each rank's program can be recorded on its own. ``simulate`` then advances the per-rank streams (one compute stream
plus one stream per communicator) until everything has run or nothing can move, and reports the operations at the
head of every stuck stream. The dependencies are the ones PyTorch's NCCL backend creates: a point-to-point operation
starts after the compute issued before it (its stream waits for the current stream), and ``wait()`` makes later
compute wait for the operation.

The reference has no counterpart (its pipeline runtime is not wired to a trainer, distributed/pipeline_runtime.py:303-471).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn

from .pipeline_runtime import PipelineParallelConfig, PipelineSchedule, PipelineScheduleType


@dataclass
class Op:
    kind: str                       # "compute" | "send" | "recv"
    stream: tuple                   # ("compute",) or the communicator key
    peer: int = -1
    label: Optional[tuple] = None
    deps: List[int] = field(default_factory=list)   # indices (into the rank's op list) that must finish first
    done: bool = False
    note: str = ""
    action: str = ""                # compute ops: "FWD" | "BWD" | "BWD_INPUT" | "BWD_WEIGHT"
    t_end: float = 0.0              # finish time in the timed replay


class RecordingTransport:
    """Stands in for the executor's transport: returns zero buffers at once and writes down what was asked for."""

    def __init__(self, sched_ref: list, chan_key=None):
        self._sched = sched_ref      # one-element list, filled after the schedule object exists
        self._chan_key = chan_key    # optional override of the executor's channel -> communicator map
        self.ops: List[Op] = []
        self._last_compute: Optional[int] = None
        self._waited: List[int] = []     # receives waited for since the last compute op

    def _p2p(self, kind_op: str, kind: str, sender: int, receiver: int, peer: int, label) -> int:
        deps = [self._last_compute] if self._last_compute is not None else []
        self.ops.append(Op(kind_op, self._key(kind, sender, receiver), peer, label, deps))
        return len(self.ops) - 1

    def _key(self, kind, sender, receiver):
        if self._chan_key is not None:
            return self._chan_key(kind, sender, receiver)
        return self._sched[0]._chan_key(kind, sender, receiver)

    def post_recv(self, kind, peer, label, shape, dtype, device):
        idx = self._p2p("recv", kind, peer, self._sched[0].rank, peer, label)
        return idx, torch.zeros(shape, dtype=dtype)

    def wait_recv(self, handle):
        idx, buf = handle
        self._waited.append(idx)
        return buf

    def send(self, kind, dst_rank, tensor, label):
        return [self._p2p("send", kind, self._sched[0].rank, dst_rank, dst_rank, label)]

    def wait_sends(self, works):
        pass

    def compute(self, action) -> None:
        deps = list(self._waited)
        if self._last_compute is not None:
            deps.append(self._last_compute)
        self._waited = []
        self.ops.append(Op("compute", ("compute",), deps=deps, action=action.type.name,
                           note=f"{action.type.name} s{action.stage} mb{action.microbatch}"))
        self._last_compute = len(self.ops) - 1


class _SimStage(nn.Module):
    def __init__(self, last: bool):
        super().__init__()
        self.w = nn.Parameter(torch.ones(()))
        self.last = last

    def forward(self, x, labels=None, **kw):
        y = x.float() * self.w
        return {"loss": y.mean()} if self.last else y


def trace_rank(schedule, p: int, m: int, rank: int, prefetch: Optional[int] = None, chan_key=None) -> List[Op]:
    """The operations rank ``rank`` issues in one step of ``schedule`` with ``p`` ranks and ``m`` microbatches.
    ``chan_key(kind, sender, receiver)`` replaces the executor's assignment of channels to communicators."""
    from ..ops import gemm as gemm_ops

    split_mode = gemm_ops.SPLIT_MODE
    try:
        ref: list = [None]
        tr = RecordingTransport(ref, chan_key)
        cfg = PipelineParallelConfig(degree=p, schedule=PipelineScheduleType(schedule), num_microbatches=m)
        sched = PipelineSchedule([nn.Identity(), nn.Identity()], None, cfg, num_microbatches=m, hidden_shape=(1, 1, 1), hidden_dtype=torch.float32,
                                 transport=tr, placement=(p, rank))
        ref[0] = sched
        if prefetch is not None:
            sched.prefetch = prefetch
        sched.stage_of = {a.stage: _SimStage(sched._last(a.stage)) for a in sched.actions if a.stage is not None}
        x = torch.ones(m, 1, 1)
        sched.step(x, target=x)
        return tr.ops
    finally:
        gemm_ops.SPLIT_MODE = split_mode


def simulate(programs: List[List[Op]], cost: Optional[Dict[str, float]] = None) -> Tuple[bool, List[str]]:
    """Advance all ranks' streams under NCCL's rules. Returns ``(finished, stuck)`` where ``stuck`` describes the head
    of every stream that could not move. With ``cost`` (durations per compute action name plus ``"p2p"``) every
    operation also gets a finish time ``t_end``: it starts when its stream is free and its dependencies (and, for a
    transfer, the peer's side) are ready."""
    n = len(programs)
    cost = cost or {}
    free: List[Dict[tuple, float]] = [dict() for _ in range(n)]

    def t_ready(r, i):
        op = programs[r][i]
        return max([free[r].get(op.stream, 0.0)] + [programs[r][d].t_end for d in op.deps])

    streams: List[Dict[tuple, List[int]]] = []
    for ops in programs:
        by: Dict[tuple, List[int]] = {}
        for i, op in enumerate(ops):
            by.setdefault(op.stream, []).append(i)
        streams.append(by)
    heads = [{k: 0 for k in by} for by in streams]

    def head(r, k):
        q, h = streams[r][k], heads[r][k]
        return q[h] if h < len(q) else None

    def ready(r, i):
        return all(programs[r][d].done for d in programs[r][i].deps)

    # the k-th send from a to b on a communicator matches the k-th receive that b posted for a on it
    def partner(r, i):
        op = programs[r][i]
        same = [j for j in streams[r][op.stream] if programs[r][j].kind == op.kind and programs[r][j].peer == op.peer]
        k = same.index(i)
        other_kind = "recv" if op.kind == "send" else "send"
        cand = [j for j in streams[op.peer].get(op.stream, [])
                if programs[op.peer][j].kind == other_kind and programs[op.peer][j].peer == r]
        return cand[k] if k < len(cand) else None

    progress = True
    while progress:
        progress = False
        for r in range(n):
            for k in streams[r]:
                i = head(r, k)
                if i is None or not ready(r, i):
                    continue
                op = programs[r][i]
                if op.kind == "compute":
                    op.t_end = t_ready(r, i) + cost.get(op.action, 0.0)
                    free[r][k] = op.t_end
                    op.done = True
                    heads[r][k] += 1
                    progress = True
                    continue
                j = partner(r, i)
                if j is None:
                    continue
                if head(op.peer, op.stream) == j and ready(op.peer, j):
                    if programs[op.peer][j].label != op.label:     # NCCL matches by order: the labels must agree
                        return False, [f"rank {r} {op.kind} {op.label} met rank {op.peer} "
                                       f"{programs[op.peer][j].kind} {programs[op.peer][j].label}"]
                    end = max(t_ready(r, i), t_ready(op.peer, j)) + cost.get("p2p", 0.0)
                    op.t_end = programs[op.peer][j].t_end = end
                    free[r][k] = free[op.peer][op.stream] = end
                    op.done = programs[op.peer][j].done = True
                    heads[r][k] += 1
                    heads[op.peer][op.stream] += 1
                    progress = True
    stuck = []
    for r in range(n):
        for k in streams[r]:
            i = head(r, k)
            if i is not None:
                op = programs[r][i]
                what = op.note if op.kind == "compute" else f"{op.kind} {op.label} peer {op.peer}"
                waiting = [programs[r][d].note or f"{programs[r][d].kind} {programs[r][d].label}"
                           for d in op.deps if not programs[r][d].done]
                stuck.append(f"rank {r} stream {k}: {what}" + (f" (after {waiting})" if waiting else ""))
    return (not stuck), stuck


def check_schedule(schedule, p: int, m: int, prefetch: Optional[int] = None, chan_key=None) -> Tuple[bool, List[str]]:
    """Trace every rank of one (schedule, p, m) and simulate the step. ``(True, [])`` when every operation ran and every
    send met the receive with its own label."""
    programs = [trace_rank(schedule, p, m, r, prefetch, chan_key) for r in range(p)]
    return simulate(programs)


def timeline(schedule, p: int, m: int, *, t_fwd: float = 1.0, t_bwd: float = 2.0, t_bwd_input: Optional[float] = None,
             t_bwd_weight: Optional[float] = None, t_p2p: float = 0.0, prefetch: Optional[int] = None) -> Dict[str, float]:
    """Timed replay of one step: ``{"makespan", "bubble"}`` where ``bubble`` is the idle share of the compute streams
    (1 - busy time / (p x makespan)). A full backward costs ``t_bwd``; schedules with a B / W split charge
    ``t_bwd_input`` and ``t_bwd_weight`` (default: half of ``t_bwd`` each); a transfer occupies its two streams for
    ``t_p2p``. For GPipe and 1F1B without transfer cost this gives the closed form (p - 1) / (m + p - 1)."""
    bi = t_bwd / 2 if t_bwd_input is None else t_bwd_input
    bw = t_bwd / 2 if t_bwd_weight is None else t_bwd_weight
    cost = {"FWD": t_fwd, "BWD": t_bwd, "BWD_INPUT": bi, "BWD_WEIGHT": bw, "p2p": t_p2p}
    programs = [trace_rank(schedule, p, m, r, prefetch) for r in range(p)]
    ok, stuck = simulate(programs, cost)
    if not ok:
        raise RuntimeError(f"schedule does not complete: {stuck[:3]}")
    makespan = max(op.t_end for ops in programs for op in ops)
    busy = sum(cost.get(op.action, 0.0) for ops in programs for op in ops if op.kind == "compute")
    return {"makespan": makespan, "bubble": 1.0 - busy / (p * makespan)}


def recommend(p: int, m: int, *, t_fwd: float = 1.0, t_bwd: float = 2.0, t_p2p: float = 0.0,
              schedules=("1F1B", "Interleaved1F1B", "LoopedBFS", "InterleavedZeroBubble", "ZBVZeroBubble", "DualPipe")):
    """Schedules ranked by replayed step time for measured per-rank costs: ``t_fwd`` / ``t_bwd`` are the forward and
    backward time of one micro-batch through *all* layers of a rank (a schedule with two chunks per rank is charged
    half per action; DualPipe's two stage copies each hold a whole rank's share), ``t_p2p`` one activation transfer.
    Returns ``[(name, makespan, bubble), ...]``, best first; a schedule that cannot run with these sizes (DualPipe and
    an odd micro-batch count) is left out."""
    out = []
    for name in schedules:
        st = PipelineScheduleType(name)
        chunks = 1 if (st.is_single_stage or st == PipelineScheduleType.dualpipe) else 2
        if st == PipelineScheduleType.dualpipe and m % 2:
            continue
        try:
            t = timeline(name, p, m, t_fwd=t_fwd / chunks, t_bwd=t_bwd / chunks, t_p2p=t_p2p)
        except Exception:  # noqa: BLE001  (sizes the generator refuses)
            continue
        out.append((name, t["makespan"], t["bubble"]))
    return sorted(out, key=lambda x: x[1])
