"""Host-side model of the flag protocol the fused expert-parallel kernels use, for testing it under arbitrary
interleavings without a GPU.

The device protocol (``csrc/moe.cu``, ``csrc/gemm_sm100.cu``, ``ops/moe.py``): every rank owns receive regions
``[local expert][source rank]``; a step has an epoch ``e`` (monotone). Per MoE layer and direction

1. *dispatch*: rank ``s`` stores its rows into region ``[.., s]`` of every destination, then releases
   ``dispatch_flags[s] = e`` on that destination (release store after a system fence);
2. *expert GEMM*: a destination tile of source ``s`` waits (bounded) for ``dispatch_flags[s] >= e`` (acquire), computes,
   stores its output rows into the source's return buffer, and the CTA that finishes the last tile destined to ``s``
   releases ``combine_flags[me] = e`` on rank ``s``;
3. *combine*: rank ``s`` waits (bounded) for ``combine_flags[d] >= e`` from every destination ``d`` it sent rows to,
   then reduces its return buffer.

Buffers are reused by the next epoch without clearing, so the only thing that keeps a reader from seeing rows of the
previous epoch is the flag order. The simulator runs the ranks as generators, lets a seeded scheduler pick which rank
advances at every memory operation, tags every stored row with ``(source, epoch)`` and checks at every read that the
tag is the expected one. Faults are injected on the host: a rank that never releases a flag (its peers' waits must
run out and report, not spin forever), or a flag released before the stores (the checker must see a stale row).

There is nothing like this in the reference (its dispatch is four blocking NCCL collectives, model/moe.py:396-497).
"""
from __future__ import annotations

import random
from dataclasses import dataclass, field
from typing import Dict, Generator, List, Optional, Tuple


class StaleRead(AssertionError):
    """A reader saw a row that was not written by the expected source in the expected epoch."""


@dataclass
class RankMemory:
    """The symmetric buffers of one rank."""

    n: int
    recv: Dict[int, Tuple[int, int]] = field(default_factory=dict)      # source -> tag (source, epoch) of its region
    ret: Dict[int, Tuple[int, int]] = field(default_factory=dict)       # destination -> tag of the returned rows
    dispatch_flags: List[int] = field(default_factory=list)
    combine_flags: List[int] = field(default_factory=list)
    status: int = 0                                                       # 0 ok, 2 = a flag wait ran out

    def __post_init__(self):
        self.dispatch_flags = [0] * self.n
        self.combine_flags = [0] * self.n


@dataclass
class Fault:
    """Host-side fault injection. ``skip_dispatch_flag`` / ``skip_combine_flag``: (rank, epoch) that never releases the
    flag; ``early_flag``: (rank, epoch) that releases its dispatch flag *before* storing the rows (a protocol bug)."""

    skip_dispatch_flag: Optional[Tuple[int, int]] = None
    skip_combine_flag: Optional[Tuple[int, int]] = None
    early_flag: Optional[Tuple[int, int]] = None


def _rank_program(r: int, mem: List[RankMemory], epochs: int, wait_budget: int, fault: Fault) -> Generator:
    """One rank's kernels for ``epochs`` steps; yields at every point where another rank may run."""
    n = len(mem)
    for e in range(1, epochs + 1):
        # --- dispatch: stores, fence, release (or, with the injected bug, release first)
        early = fault.early_flag == (r, e)
        if early:
            for d in range(n):
                mem[d].dispatch_flags[r] = e
                yield
        for d in range(n):
            mem[d].recv[r] = (r, e)
            yield
        if not early and fault.skip_dispatch_flag != (r, e):
            for d in range(n):
                mem[d].dispatch_flags[r] = e
                yield
        # --- expert GEMM on this rank: per source, wait for its flag, read its region, push results back
        for s in range(n):
            polls = 0
            while mem[r].dispatch_flags[s] < e:
                polls += 1
                if polls > wait_budget:            # bounded wait: record and give up on this source
                    mem[r].status = 2
                    break
                yield
            else:
                tag = mem[r].recv.get(s)
                if tag != (s, e):
                    raise StaleRead(f"rank {r} epoch {e}: region of source {s} holds {tag}")
                mem[s].ret[r] = (r, e)
                yield
                if fault.skip_combine_flag != (r, e):
                    mem[s].combine_flags[r] = e
                    yield
        # --- combine: wait for every destination, read the returned rows
        for d in range(n):
            polls = 0
            while mem[r].combine_flags[d] < e:
                polls += 1
                if polls > wait_budget:
                    mem[r].status = 2
                    break
                yield
            else:
                tag = mem[r].ret.get(d)
                if tag != (d, e):
                    raise StaleRead(f"rank {r} epoch {e}: rows returned by {d} hold {tag}")
        if mem[r].status:
            return                                  # the host reads the status word and stops the job
        yield


def simulate(n_ranks: int, epochs: int, seed: int, fault: Optional[Fault] = None, wait_budget: int = 10_000) -> List[int]:
    """Run the protocol under one random interleaving; returns every rank's status word. Raises ``StaleRead`` when a
    reader could observe a row of the wrong epoch."""
    rng = random.Random(seed)
    mem = [RankMemory(n_ranks) for _ in range(n_ranks)]
    progs = {r: _rank_program(r, mem, epochs, wait_budget, fault or Fault()) for r in range(n_ranks)}
    steps = 0
    while progs:
        r = rng.choice(list(progs))
        # bursts: let the chosen rank run a random number of operations, so that both fine and coarse interleavings occur
        for _ in range(rng.choice((1, 1, 2, 5, 40))):
            try:
                next(progs[r])
            except StopIteration:
                del progs[r]
                break
        steps += 1
        if steps > 5_000_000:
            raise RuntimeError("simulation did not terminate: an unbounded wait")
    return [m.status for m in mem]
