"""Pipeline-parallel runtime: model splitting, a schedule executor on NCCL/gloo p2p, gradient
clipping across stages (reference: distributed/pipeline_runtime.py:55-534).

The reference wraps ``torch.distributed.pipelining`` and a sequential DualPipe placeholder; neither
is wired to its Trainer. Here one executor runs any per-rank action list produced by
``pipeline_parallel`` (GPipe, 1F1B, Zero-Bubble with B/W split, DualPipe with two stage copies per
rank). Activations and gradients move with non-blocking ``batch_isend_irecv`` on the PP group:

* every incoming channel (peer, activation | gradient) is a FIFO in the *sender's* order, derived from the sender's
  action list, and the executor keeps ``prefetch`` receives of each channel posted ahead of the action that consumes
  them, so a transfer runs under the compute of earlier actions (NCCL matches point-to-point messages by order, not
  by tag, so receives must be posted in the order the peer sends);
* every directed channel (activation | gradient, sender, receiver) has its own two-rank communicator, so a receive
  that is posted early never sits in front of another channel's operations on one NCCL stream
  (``pipeline_sim`` replays every schedule under NCCL's ordering rules on the host);
* a zero-bubble B action runs the backward pass with every weight-gradient GEMM deferred (``ops.gemm.defer_wgrad``)
  and the W action runs them later.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from enum import Enum, StrEnum  # noqa: F401  (StrEnum: a name the reference module exposes)
from typing import Callable, Dict, List, Optional, Sequence

import torch
import torch.distributed as dist
import torch.nn as nn

from .pipeline_parallel import (Action, DualPipeSchedule, GPipeSchedule, InterleavedSchedule,
                                OneForwardOneBackwardSchedule, ScheduleType, ZeroBubbleSchedule,
                                compute_bubble_fraction)  # noqa: F401


from ..models.parallel_adapter import EMBED_ATTRS, HEAD_ATTRS  # noqa: E402,F401  (re-exported as in the reference)

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


class _CallableInt(int):
    """An int that may also be called (returns itself): lets one attribute serve as a property and as a method."""

    def __call__(self) -> int:
        return int(self)


@dataclass
class PipelineParallelConfig:
    degree: int = 1
    schedule: PipelineScheduleType = PipelineScheduleType.single_1F1B
    split_points: Optional[List[int]] = None
    num_microbatches: Optional[int] = None
    style: PipelineSplitStyle = PipelineSplitStyle.loop

    @property
    def stages_per_rank(self) -> "_CallableInt":
        """1 for GPipe / 1F1B, else 2. Reads as a number (the reference's property,
        distributed/pipeline_runtime.py:97-99) and may also be called."""
        return _CallableInt(1 if PipelineScheduleType(self.schedule).is_single_stage else 2)

    @property
    def is_single_stage(self) -> bool:
        return PipelineScheduleType(self.schedule).is_single_stage

    @property
    def total_stages(self) -> int:
        """``degree x stages_per_rank`` as in the reference (distributed/pipeline_runtime.py:101-103); the number of
        *distinct* model stages, which is ``degree`` under DualPipe, is ``num_stages()``."""
        return self.degree * int(self.stages_per_rank)

    @property
    def split_style(self) -> PipelineSplitStyle:
        if PipelineScheduleType(self.schedule) == PipelineScheduleType.zbv_zero_bubble:
            return PipelineSplitStyle.v
        return PipelineSplitStyle(self.style)

    def num_stages(self) -> int:
        """Number of distinct model stages. DualPipe keeps ``degree`` stages and gives every rank two of them (its own
        and its mirror's copy); the other two-stage schedules cut the model into ``2 * degree`` stages."""
        if PipelineScheduleType(self.schedule) == PipelineScheduleType.dualpipe:
            return self.degree
        return self.degree * self.stages_per_rank()

    def get_split_points(self, n_layers: int) -> List[int]:
        if self.split_points is not None:
            return list(self.split_points)
        return [hi for _, hi in stage_layer_ranges(n_layers, self.num_stages())[:-1]]

    def stage_ids_this_rank(self, pp_rank: int, num_stages: Optional[int] = None) -> List[int]:
        """``num_stages`` is accepted for the reference's signature (distributed/pipeline_runtime.py); the count
        follows from the schedule and the degree."""
        n, spr = self.degree, self.stages_per_rank()
        if spr == 1:
            return [pp_rank]
        if PipelineScheduleType(self.schedule) == PipelineScheduleType.dualpipe:
            return [pp_rank, n - 1 - pp_rank]       # direction 0: stage r; direction 1: the mirror rank's stage
        if PipelineScheduleType(self.schedule) == PipelineScheduleType.zbv_zero_bubble or \
                self.style == PipelineSplitStyle.v:
            return [pp_rank, self.num_stages() - 1 - pp_rank]
        return [pp_rank + s * n for s in range(spr)]


def split_model(model: nn.Module, pp_mesh=None, pp_config: Optional[PipelineParallelConfig] = None, *, device=None,
                pp_rank: Optional[int] = None, pp_group=None):
    """One module per stage owned by this rank: a deep copy of the model trimmed to the stage's
    layers (embeddings only on the first stage, head only on the last). ``pp_mesh``: the pipeline mesh or group.
    Called in the reference's keyword form ``split_model(model, pp_config=, pp_rank=, device=, pp_group=)``
    (distributed/pipeline_runtime.py:209-260) it returns the reference's pair ``(stages, model_chunks)``; a stage *is*
    its module here, so both are the same list, ready for ``PipelineSchedule(stages, ...)`` and for the optimizer."""
    assert pp_config is not None, "split_model needs pp_config"
    reference_form = pp_mesh is None and pp_rank is not None
    if pp_mesh is None:
        pp_mesh = pp_group
    group = pp_mesh.get_group() if hasattr(pp_mesh, "get_group") else pp_mesh
    if pp_rank is None:
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
        m._direction = len(stages)
        stages.append(m)
    return (stages, list(stages)) if reference_form else stages


class PipelineStages(nn.Module):
    """The stage modules one rank owns under a schedule with more than one stage per rank (interleaved, zero-bubble
    V, DualPipe). Behaves like a model for optimizers, checkpoints and the ``apply_*`` hooks; ``Trainer`` hands
    ``.stages`` to ``PipelineSchedule``. Under DualPipe the second entry is a *copy* of the mirror rank's stage: its
    gradients are summed with that rank's after every step (``sync_twin_grads``) and both copies take the same update."""

    def __init__(self, stages: Sequence[nn.Module], pp_group, pp_config: "PipelineParallelConfig"):
        super().__init__()
        self.stages = nn.ModuleList(stages)
        self._pp_enabled = True
        self._pp_group = pp_group
        self._pp_config = pp_config
        self.d_model = getattr(stages[0], "d_model", None)
        self.vocab_size = getattr(stages[0], "vocab_size", None)

    def forward(self, *a, **k):
        raise RuntimeError("a PipelineStages container is run by PipelineSchedule (Trainer does that), not called")

    def __getattr__(self, name):
        if name.startswith("apply_"):
            stages = super().__getattr__("stages")

            def fan_out(*a, **k):
                for st in stages:
                    if hasattr(st, name):
                        getattr(st, name)(*a, **k)
            return fan_out
        return super().__getattr__(name)

    @property
    def is_dualpipe(self) -> bool:
        return PipelineScheduleType(self._pp_config.schedule) == PipelineScheduleType.dualpipe


def sync_twin_grads(stages: Sequence[nn.Module], group, grad_of=None) -> None:
    """DualPipe: rank r holds stage r (direction 0) and a copy of stage p-1-r (direction 1); the mirror rank p-1-r
    holds the same two stages the other way round. Every stage therefore has one half of its gradient on each of the
    two ranks: exchange and add, so that both copies see the full gradient. One flat send + receive per rank."""
    p, r = dist.get_world_size(group), dist.get_rank(group)
    partner = p - 1 - r
    grad_of = grad_of or (lambda q: q.grad)
    order = sorted(stages, key=lambda st: st._stage_id)            # both ranks hold stages {r, p-1-r}: same order
    if partner == r:                                                # odd p, middle rank: both copies are local
        a, b = stages
        for (_, qa), (_, qb) in zip(a.named_parameters(), b.named_parameters()):
            ga, gb = grad_of(qa), grad_of(qb)
            if ga is not None and gb is not None:
                tot = ga + gb
                ga.copy_(tot)
                gb.copy_(tot)
        return
    grads = [grad_of(q) for st in order for q in st.parameters()]
    grads = [g for g in grads if g is not None]
    if not grads:
        return
    flat = torch.cat([g.reshape(-1).float() for g in grads])
    other = torch.empty_like(flat)
    peer = dist.get_global_rank(group, partner)
    for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, flat, peer, group=group),
                                     dist.P2POp(dist.irecv, other, peer, group=group)]):
        w.wait()
    flat += other
    off = 0
    for g in grads:
        g.copy_(flat[off:off + g.numel()].view_as(g))
        off += g.numel()


def sync_twin_router_counts(stages: Sequence[nn.Module], group) -> None:
    """DualPipe: the two copies of a stage each route half of the micro-batches, so the per-step load counts of their
    routers (the input of the DeepSeek-V3 bias update) are halves as well. Exchange and add them with the mirror rank,
    in stage order, so that both copies update their biases from the whole step and stay identical."""
    p, r = dist.get_world_size(group), dist.get_rank(group)
    partner = p - 1 - r
    order = sorted(stages, key=lambda st: st._stage_id)

    def counters(st):
        out = []
        for m in st.modules():
            if hasattr(m, "_tokens_per_expert_this_batch") and getattr(m, "score_bias", None) is not None:
                out += [m._tokens_per_expert_this_batch, m._total_tokens_this_batch]
        return out

    if partner == r:                       # odd p, middle rank: both copies are local
        for a, b in zip(counters(stages[0]), counters(stages[1])):
            tot = a + b
            a.copy_(tot)
            b.copy_(tot)
        return
    bufs = [c for st in order for c in counters(st)]
    if not bufs:
        return
    flat = torch.cat([c.reshape(-1).to(torch.float64) for c in bufs])
    other = torch.empty_like(flat)
    peer = dist.get_global_rank(group, partner)
    for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, flat, peer, group=group),
                                     dist.P2POp(dist.irecv, other, peer, group=group)]):
        w.wait()
    flat += other
    off = 0
    for c in bufs:
        c.copy_(flat[off:off + c.numel()].view_as(c).to(c.dtype))
        off += c.numel()


# ------------------------------------------------------------------ executor
class _P2PTransport:
    """How the executor moves a message: ``batch_isend_irecv`` on the channel's communicator. The executor talks to
    this object only, so the same ``step()`` can be replayed against a recording transport
    (``pipeline_sim.RecordingTransport``) that checks the order of operations under NCCL's rules without a GPU."""

    def __init__(self, sched: "PipelineSchedule"):
        self.s = sched

    def post_recv(self, kind: str, peer: int, label: tuple, shape, dtype, device):
        buf = torch.empty(shape, dtype=dtype, device=device)
        tag = label[2] + (10000 if kind == "grad" else 0) + 100 * label[1]
        works = dist.batch_isend_irecv([dist.P2POp(dist.irecv, buf, self.s._global(peer),
                                                   group=self.s._chan_group(kind, peer, self.s.rank), tag=tag)])
        return buf, works

    def wait_recv(self, handle):
        buf, works = handle
        for w in works:
            w.wait()
        return buf

    def send(self, kind: str, dst_rank: int, tensor: torch.Tensor, label: tuple):
        tag = label[2] + (10000 if kind == "grad" else 0) + 100 * label[1]
        return dist.batch_isend_irecv([dist.P2POp(dist.isend, tensor, self.s._global(dst_rank),
                                                  group=self.s._chan_group(kind, self.s.rank, dst_rank), tag=tag)])

    def wait_sends(self, works):
        for w in works:
            w.wait()

    def compute(self, action) -> None:   # marks where an action's kernels are issued (used by the recorder)
        pass


@dataclass
class _MB:
    inp: Optional[torch.Tensor] = None
    out: Optional[torch.Tensor] = None
    loss: Optional[torch.Tensor] = None
    grad_in: Optional[torch.Tensor] = None
    aux: Optional[torch.Tensor] = None   # auxiliary (router) loss of a stage that is not the last one


class PipelineSchedule:
    """Runs one training step of a pipeline schedule on this rank.

    ``stages``: the stage module(s) this rank owns (``split_model``). Each is called as
    ``stage(x)`` and must return the hidden state, or - on the last stage, given ``target`` - a dict
    with ``"loss"`` (the built-in ``Transformer`` does both). ``loss_fn(output, target)`` overrides that.
    ``step(inputs, target=)`` takes the full local batch, splits it into microbatches, executes this
    rank's action list and returns the mean loss on the rank holding the last stage (else ``None``).
    """

    def __init__(self, stages: Sequence[nn.Module], pp_mesh=None, pp_config: Optional[PipelineParallelConfig] = None, *,
                 num_microbatches: Optional[int] = None, loss_fn: Optional[Callable] = None,
                 hidden_shape: Optional[Sequence[int]] = None, hidden_dtype: Optional[torch.dtype] = None,
                 transport=None, placement: Optional[tuple] = None, stages_reverse: Optional[Sequence[nn.Module]] = None):
        """``transport`` / ``placement=(p, rank)``: run this rank's program without a process group, against a
        transport that records instead of sending (``pipeline_sim``). The reference's keyword form
        ``PipelineSchedule(stages=, pp_config=, loss_fn=, num_microbatches=, stages_reverse=)``
        (distributed/pipeline_runtime.py) works too: without ``pp_mesh`` the pipeline spans the default process group
        and ``stages_reverse`` (DualPipe's second direction) is appended to ``stages``."""
        assert pp_config is not None, "PipelineSchedule needs pp_config"
        if stages_reverse:
            stages = list(stages) + list(stages_reverse)
        if pp_mesh is None and placement is None and dist.is_available() and dist.is_initialized():
            pp_mesh = dist.group.WORLD
        self.stages = list(stages)
        self.group = pp_mesh.get_group() if hasattr(pp_mesh, "get_group") else pp_mesh
        self.cfg = pp_config
        if placement is not None:
            self.p, self.rank = placement
        else:
            self.p = dist.get_world_size(self.group) if self.group is not None else 1
            self.rank = dist.get_rank(self.group) if self.group is not None else 0
        self.transport = transport if transport is not None else _P2PTransport(self)
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
        elif st == PipelineScheduleType.looped_bfs:
            gen = InterleavedSchedule(self.p, self.m, v=2, placement="loop", order="bfs")
        else:  # Interleaved1F1B
            gen = InterleavedSchedule(self.p, self.m, v=2, placement="loop")
        self.generator = gen
        self.all_actions: List[List[Action]] = gen.generate_schedule()
        self.actions: List[Action] = self.all_actions[self.rank]
        self.prefetch = 2   # receives of every incoming channel kept posted ahead of their use
        self.split_w = any(a.type == ScheduleType.BWD_WEIGHT for a in self.actions)
        if self.split_w:
            from ..ops import gemm as gemm_ops

            gemm_ops.SPLIT_MODE = True   # every linear goes through the autograd function with deferrable wgrad
        self.total_stages = getattr(gen, "total_stages", 2 * self.p if self.dual else self.p)
        if self.dual:
            # direction 1 is a second copy of the pipeline: schedule stage p+s holds model stage s
            self.stage_of = {self.rank: self.stages[0], self.p + (self.p - 1 - self.rank): self.stages[-1]}
        else:
            self.stage_of = {getattr(s, "_stage_id", self.rank): s for s in self.stages}
        self._chan_groups = self._make_channel_groups() if (self.group is not None and dist.is_initialized() and
                                                            placement is None) else {}
        self.channels = self._incoming_channels()

    # -- helpers
    def _first(self, stage: int) -> bool:
        return stage in (0, self.p) if self.dual else stage == 0

    def _last(self, stage: int) -> bool:
        return stage in (self.p - 1, 2 * self.p - 1) if self.dual else stage == self.total_stages - 1

    def _rank_of(self, stage: int) -> int:
        return self.generator.rank_of_stage(stage)

    def _global(self, r: int) -> int:
        return dist.get_global_rank(self.group, r) if self.group is not None else r

    # -- point-to-point plumbing ---------------------------------------------------------------------------------
    def _make_channel_groups(self):
        """One two-rank communicator per directed channel (activation | gradient, sender, receiver) that the schedule
        uses. On NCCL all operations of a communicator run on one stream per rank in issue order and complete only
        when the peer's matching operation has reached the head of its stream, so a communicator shared by two
        channels lets a receive that was posted early hold back an unrelated send behind it; replaying the schedules
        under those rules (``pipeline_sim``) shows DualPipe on three or more ranks, the V placement on four and the
        looped placements on an odd number of ranks standing still with communicators shared by sender parity. With
        one communicator per directed channel each stream carries one FIFO whose two ends agree on the order, and
        only a cyclic schedule could block. ``new_group`` is collective over the whole job, so every rank creates the
        groups of every pipeline group, in one order."""
        if self.group is None or self.p <= 1:
            return {}
        mine = [dist.get_global_rank(self.group, r) for r in range(self.p)]
        every = [None] * dist.get_world_size()
        dist.all_gather_object(every, mine)
        keys = sorted({self._chan_key(kind, r, dst) for r in range(self.p) for kind, dst, _ in self._sends_of(r)})
        out = {}
        for ranks in sorted({tuple(x) for x in every}):
            for key in keys:
                _, a, b = key
                g = dist.new_group(sorted((ranks[a], ranks[b])))
                if tuple(mine) == ranks and self.rank in (a, b):
                    out[key] = g
        # Create the NCCL communicators now, in the same (sorted) order on every rank. Creation is collective and
        # blocking and would otherwise happen at each group's first send or receive, which the ranks of a pipeline
        # reach in different orders: each would wait inside the creation of a communicator that its peer has not
        # reached yet. In one global order the smallest unfinished key can always complete, so this cannot block.
        # The point-to-point operations are issued through ``batch_isend_irecv``, which uses the group's collective
        # communicator, so one small all-reduce per group creates the communicator they use.
        if out and dist.get_backend(self.group) == "nccl":
            warm = torch.zeros(1, device=self._device())
            # the pipeline group itself first: ``sync_twin_grads`` uses it pairwise and the middle rank of an odd
            # pipeline takes no part there, so its communicator must exist before
            dist.all_reduce(warm, group=self.group)
            for key in sorted(out):
                dist.all_reduce(warm, group=out[key])
            torch.cuda.synchronize(warm.device)
        return out

    @staticmethod
    def _chan_key(kind: str, sender_rank: int, receiver_rank: int) -> tuple:
        """Which communicator carries the messages of ``kind`` from ``sender_rank`` to ``receiver_rank``."""
        return (kind, sender_rank, receiver_rank)

    def _chan_group(self, kind: str, sender_rank: int, receiver_rank: int):
        return self._chan_groups.get(self._chan_key(kind, sender_rank, receiver_rank), self.group)

    def _sends_of(self, rank: int) -> List[tuple]:
        """(kind, destination rank, label) of every message ``rank`` sends, in its action order."""
        out = []
        for a in self.all_actions[rank]:
            if a.type == ScheduleType.FWD and not self._last(a.stage) and self._rank_of(a.stage + 1) != rank:
                out.append(("act", self._rank_of(a.stage + 1), ("act", a.stage + 1, a.microbatch)))
            elif a.type in (ScheduleType.BWD, ScheduleType.BWD_INPUT) and not self._first(a.stage) and \
                    self._rank_of(a.stage - 1) != rank:
                out.append(("grad", self._rank_of(a.stage - 1), ("grad", a.stage - 1, a.microbatch)))
        return out

    def _incoming_channels(self) -> Dict[tuple, List[tuple]]:
        """{(peer, kind): labels in the order the peer sends them} for the messages addressed to this rank."""
        ch: Dict[tuple, List[tuple]] = {}
        for peer in range(self.p):
            if peer == self.rank:
                continue
            for kind, dst, label in self._sends_of(peer):
                if dst == self.rank:
                    ch.setdefault((peer, kind), []).append(label)
        return ch

    def evaluate(self, inputs: torch.Tensor, target: Optional[torch.Tensor] = None, **kwargs):
        """Forward-only pass of the whole pipeline without gradients (validation): every rank runs the forward actions
        of its schedule in their order, activations travel as in training, and the rank holding the last stage returns
        the mean loss (the others ``None``)."""
        with torch.no_grad():
            return self.step(inputs, target, _forward_only=True, **kwargs)

    def step(self, inputs: torch.Tensor, target: Optional[torch.Tensor] = None, _forward_only: bool = False, **kwargs):
        from ..ops import gemm as gemm_ops

        m = self.m
        in_chunks = list(inputs.chunk(m, dim=0)) if inputs is not None else [None] * m
        tg_chunks = list(target.chunk(m, dim=0)) if target is not None else [None] * m
        state: Dict[tuple, _MB] = {}
        pending_send: list = []
        keepalive: list = []  # tensors of in-flight sends
        local_box: Dict[tuple, torch.Tensor] = {}  # hand-off between two stages of this rank
        wqueues: Dict[tuple, list] = {}            # deferred weight-gradient GEMMs per (stage, microbatch)
        losses: List[torch.Tensor] = []
        hs, hd = self.hidden_shape, self.hidden_dtype
        channels = {k: list(v) for k, v in self.channels.items() if not (_forward_only and k[1] == "grad")}
        nxt = {k: 0 for k in channels}              # next message of the channel to post a receive for
        posted: Dict[tuple, tuple] = {}              # label -> (buffer, works, channel)
        outstanding = {k: 0 for k in channels}

        def post_next(ch):
            peer, kind = ch
            if hs is None:
                raise RuntimeError("hidden_shape is required on stages that receive activations")
            label = channels[ch][nxt[ch]]
            nxt[ch] += 1
            posted[label] = (self.transport.post_recv(kind, peer, label, hs, hd, self._device()), ch)
            outstanding[ch] += 1

        def prefetch():
            for ch in channels:
                while outstanding[ch] < self.prefetch and nxt[ch] < len(channels[ch]):
                    post_next(ch)

        def receive(label, ch):
            while label not in posted:      # post in the sender's order until this message's receive is out
                post_next(ch)
            handle, _ = posted.pop(label)
            buf = self.transport.wait_recv(handle)
            outstanding[ch] -= 1
            return buf

        def send(kind, tensor, dst_stage, label):
            keepalive.append(tensor.detach().contiguous())
            pending_send.extend(self.transport.send(kind, self._rank_of(dst_stage), keepalive[-1], label))

        for a in self.actions:
            if a.type == ScheduleType.IDLE or (_forward_only and a.type != ScheduleType.FWD):
                continue
            if hs is not None:
                prefetch()
            stage_mod = self.stage_of[a.stage]
            key = (a.stage, a.microbatch)
            if a.type == ScheduleType.FWD:
                mb = state.setdefault(key, _MB())
                if self._first(a.stage):
                    x = in_chunks[a.microbatch]
                elif self._rank_of(a.stage - 1) == self.rank:  # previous stage lives on this rank too
                    x = local_box.pop(("act", a.stage, a.microbatch)).requires_grad_(not _forward_only)
                else:
                    x = receive(("act", a.stage, a.microbatch), (self._rank_of(a.stage - 1), "act"))
                    x.requires_grad_(not _forward_only)
                mb.inp = x
                self.transport.compute(a)     # everything this action waits for has been waited for
                if self._last(a.stage):
                    out = stage_mod(x, labels=tg_chunks[a.microbatch], **kwargs) if self.loss_fn is None else \
                        stage_mod(x, **kwargs)
                    if self.loss_fn is not None:
                        y = out["logits"] if isinstance(out, dict) and "logits" in out else out
                        loss = self.loss_fn(y, tg_chunks[a.microbatch])
                    else:
                        loss = out["loss"]
                    losses.append(loss.detach())     # what is reported: the cross-entropy, as in the non-pipelined step
                    if self.loss_fn is None and isinstance(out, dict) and out.get("aux_loss") is not None:
                        loss = loss + out["aux_loss"]
                    mb.loss = loss / m
                else:
                    out = stage_mod(x, **kwargs)
                    y = out["hidden_states"] if isinstance(out, dict) else out
                    mb.out = y
                    if isinstance(out, dict) and out.get("aux_loss") is not None and out["aux_loss"].requires_grad:
                        mb.aux = out["aux_loss"] / m   # back-propagated locally together with the incoming gradient
                    if hs is None:
                        hs, hd = tuple(y.shape), y.dtype
                    if self._rank_of(a.stage + 1) == self.rank:
                        local_box[("act", a.stage + 1, a.microbatch)] = y.detach().clone()
                    else:
                        send("act", y, a.stage + 1, ("act", a.stage + 1, a.microbatch))
                if _forward_only:
                    state.pop(key, None)       # nothing comes back for this micro-batch
            elif a.type in (ScheduleType.BWD, ScheduleType.BWD_INPUT):
                mb = state[key]
                if self._last(a.stage):
                    root, g = mb.loss, None
                elif self._rank_of(a.stage + 1) == self.rank:
                    root, g = mb.out, local_box.pop(("grad", a.stage, a.microbatch))
                else:
                    root, g = mb.out, receive(("grad", a.stage, a.microbatch), (self._rank_of(a.stage + 1), "grad"))
                roots, gouts = [root], [g]
                self.transport.compute(a)
                if mb.aux is not None:
                    roots.append(mb.aux)
                    gouts.append(torch.ones_like(mb.aux))
                if a.type == ScheduleType.BWD_INPUT:
                    # B: everything except the weight-gradient GEMMs, which wait in a queue for this pair's W action
                    with gemm_ops.defer_wgrad(wqueues.setdefault(key, [])):
                        torch.autograd.backward(roots, gouts)
                else:
                    torch.autograd.backward(roots, gouts)
                if not self._first(a.stage) and mb.inp.grad is not None:
                    if self._rank_of(a.stage - 1) == self.rank:
                        local_box[("grad", a.stage - 1, a.microbatch)] = mb.inp.grad
                    else:
                        send("grad", mb.inp.grad, a.stage - 1, ("grad", a.stage - 1, a.microbatch))
                state.pop(key)
            elif a.type == ScheduleType.BWD_WEIGHT:
                self.transport.compute(a)
                gemm_ops.run_deferred_wgrads(wqueues.pop(key, []))
        for q in wqueues.values():      # a schedule without W actions for some pair: nothing may be left behind
            gemm_ops.run_deferred_wgrads(q)
        self.transport.wait_sends(pending_send)
        if losses:
            return torch.stack(losses).mean()
        return None

    def loss_on_all_ranks(self, loss: Optional[torch.Tensor]) -> torch.Tensor:
        """The step's (or evaluation's) loss on every rank of the pipeline: broadcast from the rank that holds the last
        stage; under DualPipe the mean of the two directions' losses (ranks p-1 and 0)."""
        t = loss.detach().float().clone() if loss is not None else torch.zeros((), device=self._device())
        if self.group is None or self.p <= 1:
            return t
        if self.dual:
            both = t if self.rank in (0, self.p - 1) else torch.zeros_like(t)
            dist.all_reduce(both, group=self.group)
            return both / 2
        src = self._rank_of(self.total_stages - 1)
        dist.broadcast(t, dist.get_global_rank(self.group, src), group=self.group)
        return t

    def _device(self):
        for s in self.stages:
            for p in s.parameters():
                return p.device
        return torch.device("cpu")


class DualPipeScheduleRuntime(PipelineSchedule):
    """DualPipe executor: this rank owns two stage copies (one per direction); even microbatches
    enter at rank 0, odd ones at rank p-1 (reference: distributed/pipeline_runtime.py:303-397, which
    runs the phases sequentially on one direction only)."""

    def __init__(self, stages, pp_mesh=None, pp_config=None, loss_fn=None, **kw):
        """``DualPipeScheduleRuntime(stages, pp_mesh, pp_config)`` with this rank's two stage copies, or the
        reference's ``(stages_forward, stages_reverse, num_microbatches, loss_fn)``
        (distributed/pipeline_runtime.py:303-320): two lists of stages, told apart by the second argument being a list."""
        if isinstance(pp_mesh, (list, tuple, nn.ModuleList)):
            stages_reverse, num_microbatches = pp_mesh, pp_config
            stages = list(stages) + list(stages_reverse)
            pp_mesh = kw.pop("group", None)
            pp_config = PipelineParallelConfig(degree=max(len(stages) // 2, 1), schedule=PipelineScheduleType.dualpipe,
                                               num_microbatches=num_microbatches if isinstance(num_microbatches, int)
                                               else None)
        cfg = pp_config or PipelineParallelConfig(schedule=PipelineScheduleType.dualpipe)
        cfg.schedule = PipelineScheduleType.dualpipe
        if loss_fn is not None:
            kw["loss_fn"] = loss_fn
        super().__init__(stages, pp_mesh, cfg, **kw)


def clip_grad_norm_pp(parameters, max_norm=None, pp_group=None, norm_type: float = 2.0,
                      copies: int = 1, ep_group=None, *, max_grad_norm: Optional[float] = None,
                      model_parts=None) -> torch.Tensor:
    """Clip by the global norm over all pipeline stages (one scalar all-reduce over the PP group). ``copies``: how
    many ranks hold each stage (2 under DualPipe, whose twin copies carry identical gradients after
    ``sync_twin_grads``), so that every stage counts once. Composed with other dimensions every parameter still counts
    once: tensor-parallel shards (``_tp_sharded`` = their TP group) add up over that group, expert shards
    (``_ep_sharded``) over ``ep_group``, everything else is identical on those peers."""
    if model_parts is not None:
        parameters = model_parts
    parameters = list(parameters)
    if parameters and isinstance(parameters[0], nn.Module):
        # the reference's form: clip_grad_norm_pp(model_parts, pp_group, max_grad_norm, norm_type)
        # (distributed/pipeline_runtime.py): stage modules first, then the group, then the norm
        if isinstance(pp_group, (int, float)) and not isinstance(pp_group, bool):
            max_norm, pp_group = pp_group, max_norm          # positional: the group sits where max_norm is expected
        elif max_norm is not None and not isinstance(max_norm, (int, float)):
            max_norm, pp_group = None, max_norm              # group positional, the norm by keyword
        seen, flat = set(), []
        for mod in parameters:
            for q in mod.parameters():
                if id(q) not in seen:
                    seen.add(id(q))
                    flat.append(q)
        parameters = flat
    if max_grad_norm is not None:
        max_norm = max_grad_norm
    params = [p for p in parameters if p.grad is not None]
    dev = params[0].device if params else torch.device("cpu")
    if norm_type == float("inf"):
        total = torch.stack([p.grad.detach().abs().max() for p in params]).max() if params else torch.zeros((), device=dev)
        groups = {id(g): g for g in [pp_group, ep_group, *[getattr(p, "_tp_sharded", None) for p in params]]
                  if g is not None}
        for g in groups.values():
            dist.all_reduce(total, op=dist.ReduceOp.MAX, group=g)
    else:
        def sq(ps):
            return torch.stack([p.grad.detach().float().norm(norm_type) ** norm_type for p in ps]).sum() \
                if ps else torch.zeros((), device=dev)

        tp_groups = {}
        for p in params:
            g = getattr(p, "_tp_sharded", None)
            if g is not None:
                tp_groups.setdefault(id(g), (g, []))[1].append(p)
        ep_params = [p for p in params if getattr(p, "_ep_sharded", False) and getattr(p, "_tp_sharded", None) is None]
        rest = [p for p in params if getattr(p, "_tp_sharded", None) is None and not getattr(p, "_ep_sharded", False)]
        total = sq(rest)
        for g, ps in tp_groups.values():
            part = sq(ps)
            dist.all_reduce(part, group=g)
            total = total + part
        if ep_params or ep_group is not None:
            part = sq(ep_params)
            if ep_group is not None:
                dist.all_reduce(part, group=ep_group)
            total = total + part
        if pp_group is not None:
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=pp_group)
        total = (total / max(copies, 1)) ** (1.0 / norm_type)
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for p in params:
        p.grad.mul_(coef.to(p.grad.dtype))
    return total
