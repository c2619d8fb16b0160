"""Profile-driven pipeline schedule generation (reference: distributed/auto_schedule.py:30-259).

Given per-stage forward/backward/communication times and a memory budget, builds a 1F1B or
DualPipe-style per-rank schedule, simulates it with the measured costs (the same dependency
simulator that validates the hand-written generators) and reports bubble fraction, the share of
communication hidden behind compute and whether the in-flight activations fit the budget.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List

from . import pipeline_parallel as pp


@dataclass
class StageProfile:
    fwd_time: float = 1.0
    bwd_time: float = 2.0
    comm_time: float = 0.5
    mem_gb: float = 4.0


@dataclass
class AutoScheduleConfig:
    num_microbatches: int = 8
    num_stages: int = 4
    dualpipe_ratio: float = 0.0
    memory_budget_gb: float = 180.0
    overlap_comm: bool = True


@dataclass
class Action:
    type: str  # "FWD" | "BWD" | "BWD_W"
    microbatch_idx: int
    stage_idx: int
    step_idx: int


class AutoScheduleGenerator:
    def __init__(self, stage_profiles: List[StageProfile], config: AutoScheduleConfig):
        self.profiles = stage_profiles
        self.config = config
        self.p = len(stage_profiles)
        self.m = config.num_microbatches
        self.half_m = self.m // 2

    def _raw(self):
        if self.config.dualpipe_ratio > 0:
            gen = pp.DualPipeSchedule(num_stages=self.p, num_microbatches=self.m, split_w=False)
        else:
            gen = pp.OneForwardOneBackwardSchedule(self.p, self.m)
        return gen, gen.generate_schedule()

    def generate(self) -> List[List[Action]]:
        _, raw = self._raw()
        out = []
        for acts in raw:
            row = []
            for i, a in enumerate(acts):
                kind = {"FWD": "FWD", "BWD": "BWD", "BWD_INPUT": "BWD", "BWD_WEIGHT": "BWD_W"}.get(a.type.name)
                if kind:
                    row.append(Action(kind, a.microbatch, a.stage, i))
            out.append(row)
        return out

    def _simulate(self):
        gen, raw = self._raw()
        f = sum(s.fwd_time for s in self.profiles) / self.p
        b = sum(s.bwd_time for s in self.profiles) / self.p
        c = 0.0 if self.config.overlap_comm else sum(s.comm_time for s in self.profiles) / self.p
        costs = {pp.F: f + c, pp.B: b + c, pp.BI: b / 2 + c, pp.W: b / 2}
        dual = self.config.dualpipe_ratio > 0
        first = (lambda s: 0 if s < self.p else self.p) if dual else None
        last = (lambda s: self.p - 1 if s < self.p else 2 * self.p - 1) if dual else None
        return pp.validate_schedule(raw, self.p, self.m, stage_first=first, stage_last=last, costs=costs)

    def compute_bubble_fraction(self) -> float:
        return self._simulate()["bubble_fraction"]

    def compute_overlap_efficiency(self) -> float:
        """Share of the p2p time hidden behind compute: transfers are posted asynchronously, so with
        ``overlap_comm`` a transfer is exposed only where it is longer than the compute it overlaps."""
        comm = sum(s.comm_time for s in self.profiles)
        if comm == 0:
            return 1.0
        if not self.config.overlap_comm:
            return 0.0
        hidden = sum(min(s.comm_time, s.fwd_time) for s in self.profiles)
        return hidden / comm

    def validate_memory(self) -> tuple:
        """``(fits, peak_activations_gb)`` as in the reference (distributed/auto_schedule.py:249-259). 1F1B keeps at
        most ``p - rank`` microbatches of activations alive on a rank (DualPipe: about ``p + 1`` over both
        directions); the largest of those has to fit the per-GPU budget. (The reference charges every rank
        ``min(p, m)`` microbatches of the largest stage, the first rank's figure.)"""
        worst = 0.0
        for r, s in enumerate(self.profiles):
            inflight = (self.p + 1) if self.config.dualpipe_ratio > 0 else (self.p - r)
            worst = max(worst, s.mem_gb * min(inflight, self.m))
        return worst <= self.config.memory_budget_gb, worst
