"""Mixture-of-experts layer: router, capacity, expert-parallel dispatch/combine, expert MLPs
(reference: model/moe.py, whole file).

Public names and constructor signatures follow the reference. What differs, by design:

* The router statistics (per-expert counts, drop counters) stay on the device; nothing in the
  forward pass synchronises with the host on the CUDA path.
* Expert parallelism is correct for ``ep_size > 1``: expert weights are sharded (rank r owns experts
  ``[r*E/ep, (r+1)*E/ep)``), dispatch carries (row, local expert id) pairs and combine returns the
  weighted sum per token. ``NcclAllToAllDispatcher`` is the plain-collective implementation (works on
  gloo for CPU tests); ``SymmetricMemoryDispatcher`` is the fused sm_100a path that pushes rows into
  peer memory from inside the kernels (``ops/moe.py``).
* Capacity keeps the reference rule (``capacity = int(cf * T / E)``, a token over capacity for any of
  its experts is dropped whole, in index order) but is computed with prefix sums instead of a Python
  loop over experts.
* ``post_batch`` moves the DeepSeek-V3 bias *against* the load (over-loaded experts are pushed
  down); ``bias_update_sign=+1`` restores the reference's direction. The load fraction is the expert's share of
  all assignments (the shares sum to 1, so the update has zero mean); the reference divides the counts by the
  number of tokens (shares sum to top-k), which is this update with ``gamma`` times top-k plus a shift common to all
  experts - invisible to top-k selection and softmax gating, a drift under sigmoid gating.
* ``last_dropped`` / ``total_dropped`` / ``drop_rate`` count dropped *tokens*; the reference adds up the per-expert
  overflows, which counts a token once per over-full expert it chose (its rate can exceed 1): that figure is
  ``last_dropped_slots``. ``per_expert_drops`` and the adaptive-capacity estimate are the reference's.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import _lib
from .ep_runtime import AdaptiveSMAllocator, CoupledEPScheduler, EPScheduleDecision, RoutingPrefetcher  # noqa: F401


class GatingFunction(str, Enum):
    SOFTMAX = "softmax"
    SIGMOID = "sigmoid"


class MoELoadBalancingLossGranularity(str, Enum):
    LOCAL_BATCH = "local_batch"
    GLOBAL = "global"           # the reference's second member (model/moe.py:49-51)
    INSTANCE = "instance"


@dataclass
class MoERouterConfig:
    num_experts: int = 8
    top_k: int = 2
    gating_function: GatingFunction = GatingFunction.SOFTMAX
    bias_init: Optional[float] = -1.0
    bias_gamma: Optional[float] = None
    z_loss_multiplier: Optional[float] = None
    jitter_eps: Optional[float] = None
    normalize_expert_weights: Optional[str] = None
    routing_replay: bool = False
    routing_replay_mask: Optional[torch.Tensor] = None
    bias_update_sign: float = -1.0  # -1: DeepSeek-V3 direction; +1: the reference's direction


class MoERouter(nn.Module):
    """fp32 gate with bias, DeepSeek-V3 score bias, top-k softmax / sigmoid gating, aux + z loss."""

    def __init__(self, *, d_model: int, config: MoERouterConfig, device=None):
        super().__init__()
        self.config = config
        self.num_experts = config.num_experts
        self.top_k = config.top_k
        self.gate = nn.Linear(d_model, config.num_experts, bias=True, dtype=torch.float32, device=device)
        if config.bias_init is not None:
            nn.init.constant_(self.gate.bias, config.bias_init)
        if config.bias_gamma is not None:
            self.register_buffer("score_bias", torch.zeros(config.num_experts, device=device))
            self.register_buffer("_tokens_per_expert_this_batch",
                                 torch.zeros(config.num_experts, dtype=torch.long, device=device))
            self.register_buffer("_total_tokens_this_batch", torch.tensor(0, dtype=torch.long, device=device))
        else:
            self.score_bias = None
        self.routing_replay = config.routing_replay
        self._replay_mask: Optional[torch.Tensor] = config.routing_replay_mask
        self.last_counts: Optional[torch.Tensor] = None  # per-expert assignments of the last forward

    def _apply(self, fn, recurse=True):  # the gate stays fp32 under .to(bf16)
        super()._apply(fn, recurse)
        for p in (self.gate.weight, self.gate.bias):
            if p is not None and p.dtype != torch.float32:
                p.data = p.data.float()
        if self.score_bias is not None and self.score_bias.dtype != torch.float32:
            self.score_bias = self.score_bias.float()
        return self

    # -- gating variants ------------------------------------------------------------------------
    def _softmax_gating(self, logits):
        top_logits, top_idx = logits.topk(self.top_k, dim=-1)
        return F.softmax(top_logits, dim=-1), top_idx

    def _sigmoid_gating(self, logits):
        scores = torch.sigmoid(logits)
        w, idx = scores.topk(self.top_k, dim=-1)
        return w / (w.sum(dim=-1, keepdim=True) + 1e-8), idx

    def _routing_replay_gating(self, logits, mask):
        """R3 replay: restrict the choice to the experts recorded at inference time. ``mask``: the recorded expert
        *indices*, ``(B, S, K)`` or ``(N, K)`` - what the reference's ``set_replay_mask`` takes and scatters
        (model/moe.py:186-240) - or a boolean ``(..., num_experts)`` mask of allowed experts. The weights are the
        softmax of the training logits over the replayed experts, so the router still receives gradients."""
        mask = mask.to(logits.device)
        if mask.dtype != torch.bool and mask.shape[-1] == self.top_k and self.top_k != self.num_experts:
            idx = mask.reshape(-1, self.top_k).long()
            allowed = torch.zeros(idx.shape[0], self.num_experts, dtype=torch.bool, device=logits.device)
            mask = allowed.scatter_(1, idx, True)
        mask = mask.reshape(logits.shape).bool()
        masked = logits.masked_fill(~mask, float("-inf"))
        # rows whose mask allows fewer than top_k experts fall back to the unmasked logits
        enough = mask.sum(-1, keepdim=True) >= self.top_k
        masked = torch.where(enough, masked, logits)
        top_logits, top_idx = masked.topk(self.top_k, dim=-1)
        return F.softmax(top_logits, dim=-1), top_idx

    def set_replay_mask(self, mask: torch.Tensor):
        self._replay_mask = mask

    def clear_replay_mask(self):
        self._replay_mask = None

    def _load_balancing_loss(self, logits, indices):
        n_tok = logits.numel() // logits.shape[-1]
        counts = torch.zeros(self.num_experts, device=logits.device, dtype=torch.float32)
        counts.scatter_add_(0, indices.reshape(-1), torch.ones(indices.numel(), device=logits.device))
        P = F.softmax(logits.float(), dim=-1).reshape(-1, self.num_experts).mean(0)
        n = self._token_shards()
        if n > 1:
            # The rows of one batch are spread over other ranks (sequence-parallel tensor parallelism: 1 / tp of the
            # rows; context parallelism: 1 / cp of every sequence). The loss is E * sum(f * P) over *all* rows: f (token
            # fractions, no gradient) is summed over those ranks; P is a mean of per-rank means, so each rank
            # contributes f_all * P_local / n and the contributions add up - in value after the all-reduce below, in
            # gradient through the sum of the partial gradients that these layouts form anyway.
            all_counts = counts.clone()
            for g in self._token_shard_groups():
                dist.all_reduce(all_counts, group=g)
            part = self.num_experts * ((all_counts / (n_tok * n)) * P).sum() / n
            return self._sp_total(part), counts
        f = counts / n_tok
        return self.num_experts * (f * P).sum(), counts

    def _token_shard_groups(self) -> list:
        """Groups over which the rows of one batch are spread: ``_sp_group`` (set by sequence-parallel TP) and
        ``_cp_group`` (set by context parallelism). Summing over each in turn sums over their product."""
        if not (dist.is_available() and dist.is_initialized()):
            return []
        return [g for g in (getattr(self, "_sp_group", None), getattr(self, "_cp_group", None))
                if g is not None and dist.get_world_size(g) > 1]

    def _token_shards(self) -> int:
        n = 1
        for g in self._token_shard_groups():
            n *= dist.get_world_size(g)
        return n

    def _sp_total(self, part: torch.Tensor) -> torch.Tensor:
        """Value: the sum of ``part`` over the ranks that share the batch's rows; gradient: this rank's ``part`` only."""
        tot = part.detach().clone()
        for g in self._token_shard_groups():
            dist.all_reduce(tot, group=g)
        return part + (tot - part.detach())

    def forward(self, x: torch.Tensor):
        """x: (B, S, D) or (T, D) -> (weights (..., K) fp32, indices (..., K) int64, aux_loss)."""
        cfg = self.config
        if cfg.jitter_eps is not None and self.training:
            x = x + torch.randn_like(x) * cfg.jitter_eps
        replay = self.routing_replay and self._replay_mask is not None and self.training
        if _lib.on(x) and x.dtype == torch.bfloat16 and not replay and cfg.normalize_expert_weights is None:
            from ..ops import moe as moe_ops

            w, idx, aux, counts = moe_ops.route(x, self)
            n = self._token_shards()
            if n > 1:
                # the router kernels take their load statistics over this rank's rows: with the batch's rows spread
                # over other ranks (sequence-parallel TP, context parallelism) the loss is then the mean of the ranks'
                # own losses (Megatron's per-rank form) rather than the loss of the whole batch that the PyTorch path
                # below computes
                aux = self._sp_total(aux / n)
        else:
            logits = F.linear(x.float(), self.gate.weight, self.gate.bias)
            if self.score_bias is not None:
                logits = logits + self.score_bias
            if replay:
                w, idx = self._routing_replay_gating(logits, self._replay_mask)
            elif cfg.gating_function == GatingFunction.SIGMOID:
                w, idx = self._sigmoid_gating(logits)
            else:
                w, idx = self._softmax_gating(logits)
            if cfg.normalize_expert_weights == "l2":
                w = w / (w.norm(dim=-1, keepdim=True) + 1e-8)
            aux, counts = self._load_balancing_loss(logits, idx)
            if cfg.z_loss_multiplier is not None:
                z = cfg.z_loss_multiplier * torch.logsumexp(logits.float(), dim=-1).square().mean()
                n = self._token_shards()
                if n > 1:
                    z = self._sp_total(z / n)    # mean over all rows = mean of the ranks' means
                aux = aux + z
        self.last_counts = counts.detach()
        if self.score_bias is not None:
            self._update_expert_counts(idx, counts)
        return w, idx, aux

    @torch.no_grad()
    def _update_expert_counts(self, indices, counts=None):
        if counts is None:
            counts = torch.bincount(indices.reshape(-1), minlength=self.num_experts)
        self._tokens_per_expert_this_batch += counts.to(self._tokens_per_expert_this_batch)
        self._total_tokens_this_batch += indices.numel()

    @torch.no_grad()
    def post_batch(self, group=None, *, groups=None) -> None:
        """DeepSeek-V3 bias update, once per step: ``bias += sign * gamma * (load_fraction - 1/E)``. The token counts
        are summed over ``group`` (default: all ranks) or, with ``groups`` given, over each group of that list in turn
        (an empty list: no reduction). Only ranks that hold *this* layer and route other tokens belong there - the
        replica group, plus the TP group under sequence parallelism; a reduction over all ranks of a pipelined job
        would pair this layer's counts with another stage's layer."""
        if self.score_bias is None or getattr(self, "_device_side_update", False):
            return  # no bias, or the fused runtime updates all layers on the device (ops.moe.update_router_bias)
        if dist.is_available() and dist.is_initialized():
            packed = torch.cat([self._tokens_per_expert_this_batch, self._total_tokens_this_batch.reshape(1)])
            if groups is None:
                dist.all_reduce(packed, group=group)
            else:
                for g in groups:
                    dist.all_reduce(packed, group=g)
            self._tokens_per_expert_this_batch.copy_(packed[:-1])
            self._total_tokens_this_batch.copy_(packed[-1])
        total = self._total_tokens_this_batch.float().clamp_min(1.0)
        frac = self._tokens_per_expert_this_batch.float() / total
        upd = self.config.bias_update_sign * self.config.bias_gamma * (frac - 1.0 / self.num_experts)
        upd = torch.where(self._total_tokens_this_batch > 0, upd, torch.zeros_like(upd))
        self.score_bias += upd.to(self.score_bias)
        self._tokens_per_expert_this_batch.zero_()
        self._total_tokens_this_batch.zero_()


# ------------------------------------------------------------------------------------------------
# Expert-parallel dispatch
# ------------------------------------------------------------------------------------------------
class _AllToAllSingle(torch.autograd.Function):
    """``all_to_all_single`` with uneven row splits; the backward pass swaps the split lists."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits), *g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


class _CallableInt(int):
    """An int that may also be called (returns itself)."""

    def __call__(self) -> int:
        return int(self)


class TokenDispatcher:
    """Interface of an EP dispatcher.

    ``dispatch(x (T,D), expert_indices (T,K), expert_weights (T,K), num_experts, ep_size, ep_rank, ep_group)`` - the
    reference's signature (model/moe.py:335-345) - returns ``(local_x (n,D), local_weights (n,), local_indices (n,)
    local expert ids, meta)`` with rows sorted by local expert; ``combine(expert_output (n,D), combine_metadata, x,
    expert_weights, expert_indices, ep_size, ep_group)`` returns ``(T, D)``: the router-weighted sum of every token's K
    expert outputs.
    """

    def dispatch(self, x, expert_indices, expert_weights, num_experts, ep_size=1, ep_rank=None, ep_group=None):
        raise NotImplementedError

    def combine(self, expert_output, combine_metadata, x, expert_weights, expert_indices, ep_size=None, ep_group=None):
        raise NotImplementedError


class NcclAllToAllDispatcher(TokenDispatcher):
    """Plain-collective dispatcher: one counts all-to-all, rows and expert ids by
    ``all_to_all_single`` (NCCL on GPU, gloo on CPU). This is the un-fused baseline."""

    def dispatch(self, x, expert_indices, expert_weights, num_experts, ep_size=1, ep_rank=None, ep_group=None):
        indices, weights = expert_indices, expert_weights
        if not isinstance(ep_size, int):       # the former order of this package: (..., num_experts, ep_group, ep_size)
            ep_size, ep_group = (ep_rank if isinstance(ep_rank, int) else 1), ep_size
        T, K = indices.shape
        flat_e = indices.reshape(-1)
        order = torch.argsort(flat_e, stable=True)
        rows = x[order // K]
        sorted_e = flat_e[order]
        sorted_w = weights.reshape(-1)[order]
        if ep_size <= 1:
            meta = dict(order=order, T=T, K=K, ep_size=1)
            return rows, sorted_w, sorted_e, meta
        e_local = num_experts // ep_size
        send_counts = torch.bincount(sorted_e // e_local, minlength=ep_size)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts, group=ep_group)
        send_l, recv_l = send_counts.tolist(), recv_counts.tolist()
        recv_rows = _AllToAllSingle.apply(rows, recv_l, send_l, ep_group)
        ids_out = sorted_e.new_empty(sum(recv_l))
        dist.all_to_all_single(ids_out, sorted_e.contiguous(), recv_l, send_l, group=ep_group)
        w_out = _AllToAllSingle.apply(sorted_w.reshape(-1, 1), recv_l, send_l, ep_group).reshape(-1)
        local_ids = ids_out - dist.get_rank(ep_group) * e_local
        order2 = torch.argsort(local_ids, stable=True)
        meta = dict(order=order, order2=order2, send=send_l, recv=recv_l, group=ep_group, T=T, K=K,
                    ep_size=ep_size)
        return recv_rows[order2], w_out[order2], local_ids[order2], meta

    def combine(self, expert_output, combine_metadata, x, expert_weights, expert_indices, ep_size=None, ep_group=None):
        meta, weights = combine_metadata, expert_weights
        T, K = meta["T"], meta["K"]
        if meta["ep_size"] > 1:
            unsorted = torch.empty_like(expert_output)
            unsorted[meta["order2"]] = expert_output
            expert_output = _AllToAllSingle.apply(unsorted, meta["send"], meta["recv"], meta["group"])
        slot_rows = torch.empty_like(expert_output)
        slot_rows[meta["order"]] = expert_output
        w = weights.reshape(T, K, 1).to(slot_rows.dtype)
        return (slot_rows.view(T, K, -1) * w).sum(dim=1)


class SymmetricMemoryDispatcher(NcclAllToAllDispatcher):
    """Marker for the fused sm_100a path: dispatch, expert GEMMs and combine run as kernels that
    store into / read from peer memory (``ops.moe.fused_moe``). The phase API falls back to the
    collective implementation of the base class."""

    fused = True


class DeepEPDispatcher(SymmetricMemoryDispatcher):
    """The reference's optional DeepEP backend (model/moe.py:501-617) mapped onto the in-tree symmetric-memory
    kernels; ``deep_ep`` itself is not used. Its three knobs configure the fused runtime that
    ``ops.moe.build_runtime`` creates for the layers holding this dispatcher:

    * ``num_sms``: CTAs the dispatch kernel may occupy (the rest of the GPU keeps running the dense branch of a hybrid
      block or the previous GEMM's tail); ``None`` with ``adaptive=True`` asks ``AdaptiveSMAllocator`` for the
      roofline split of the layer's shapes, ``None`` otherwise means all SMs;
    * ``use_fp8_dispatch``: rows travel as e4m3 with 1x128 scales and feed the e4m3 expert GEMMs, regardless of the
      tokens-per-expert threshold of the FP8-Flow-MoE switch;
    * ``async_with_compute_stream``: kept for signature parity. The fused kernels always run in stream order with the
      compute kernels and overlap through their arrival flags, which is what the option asks DeepEP for.
    """

    def __init__(self, num_sms: Optional[int] = None, use_fp8_dispatch: bool = False,
                 async_with_compute_stream: bool = True, adaptive: bool = False):
        self.num_sms = num_sms
        self.use_fp8_dispatch = use_fp8_dispatch
        self.async_with_compute_stream = async_with_compute_stream
        self.adaptive = adaptive

    def dispatch_ctas(self, *, tokens: int, d_model: int, hidden: int, num_experts: int, top_k: int,
                      fp8: bool = False) -> int:
        """CTA budget of the dispatch kernel (0 = no limit)."""
        if self.num_sms:
            return int(self.num_sms)
        if not self.adaptive:
            return 0
        return AdaptiveSMAllocator().compute_optimal_sms(tokens, d_model, hidden, num_experts, top_k,
                                                        num_bytes_per_elem=1 if fp8 else 2)


def get_best_dispatcher() -> TokenDispatcher:
    """Fused peer-memory dispatcher on a GPU, the collective one otherwise."""
    if torch.cuda.is_available():
        return SymmetricMemoryDispatcher()
    return NcclAllToAllDispatcher()


@dataclass
class ExpertParallelConfig:
    ep_size: int = 1
    ep_group: Optional[object] = None
    dispatcher: Optional[TokenDispatcher] = None

    def __post_init__(self):
        if self.dispatcher is None:
            self.dispatcher = get_best_dispatcher()

    @property
    def ep_rank(self) -> int:
        """This rank's index in the EP group; reads as a number and may be called (a method in the reference,
        model/moe.py:660-663)."""
        if self.ep_size <= 1 or self.ep_group is None:
            return _CallableInt(0)
        return _CallableInt(dist.get_rank(self.ep_group))

    def local_experts(self, num_experts: int) -> tuple[int, int]:
        n = num_experts // max(self.ep_size, 1)
        return self.ep_rank * n, (self.ep_rank + 1) * n

    def _reference_style(self) -> bool:
        """A dispatcher written against the reference's interface takes ``(x, expert_indices, expert_weights,
        num_experts, ep_size, ep_rank, ep_group)`` and ``combine(..., ep_size, ep_group)`` (model/moe.py:335-357)."""
        import inspect

        try:
            return "ep_rank" in inspect.signature(self.dispatcher.dispatch).parameters
        except (TypeError, ValueError):
            return False

    def dispatch(self, x, expert_indices, expert_weights, num_experts):
        indices, weights = expert_indices, expert_weights
        if self._reference_style():
            return self.dispatcher.dispatch(x, indices, weights, num_experts, self.ep_size, int(self.ep_rank),
                                            self.ep_group)
        # a dispatcher written for this package's earlier interface
        return self.dispatcher.dispatch(x, indices, weights, num_experts, self.ep_group, self.ep_size)

    def combine(self, expert_output, combine_metadata, x, expert_weights, expert_indices):
        meta, weights, indices = combine_metadata, expert_weights, expert_indices
        if self._reference_style():
            return self.dispatcher.combine(expert_output, meta, x, weights, indices, self.ep_size, self.ep_group)
        return self.dispatcher.combine(expert_output, meta, x, weights, indices)


# ------------------------------------------------------------------------------------------------
# Experts
# ------------------------------------------------------------------------------------------------
class ExpertMLP(nn.Module):
    """Shared-expert SwiGLU MLP with the reference's parameters (model/moe.py:1164-1183): ``w1``, ``w3`` and ``w2`` all
    ``(hidden, d_model)``, ``forward(x) = (silu(x w1^T) * (x w3^T)) w2``. Names, shapes and registration order are the
    reference's, so model and optimizer state move between the two code bases. On CUDA in bf16 the three products run
    on the tcgen05 GEMM; ``w2`` is stored input-major, so it is handed over as a transposed copy (hidden x d_model
    elements per forward, against a GEMM over all tokens)."""

    def __init__(self, d_model: int, hidden_size: int, dtype=None, device=None, init_std: float = 0.01):
        super().__init__()
        self.d_model, self.hidden_size = d_model, hidden_size
        kw = dict(dtype=dtype, device=device)
        self.w1 = nn.Parameter(torch.empty(hidden_size, d_model, **kw))
        self.w2 = nn.Parameter(torch.empty(hidden_size, d_model, **kw))
        self.w3 = nn.Parameter(torch.empty(hidden_size, d_model, **kw))
        for w in (self.w1, self.w2, self.w3):
            nn.init.normal_(w, std=init_std)
        self._register_load_state_dict_pre_hook(self._earlier_keys_in)

    @staticmethod
    def _earlier_keys_in(state_dict, prefix, *_):
        """Checkpoints of this package written while the shared expert wrapped a ``FeedForward``
        (``ffn.w1.weight`` ..., ``w2`` output-major, plus alias entries ``w1.weight`` ...)."""
        for name in ("w1", "w2", "w3"):
            state_dict.pop(f"{prefix}{name}.weight", None)
            old = f"{prefix}ffn.{name}.weight"
            if old in state_dict:
                t = state_dict.pop(old)
                state_dict[prefix + name] = t.t() if name == "w2" else t

    def forward(self, x):
        if _lib.on(x) and x.dtype == torch.bfloat16 and self.w1.dtype == torch.bfloat16:
            from ..ops import activation as act_ops
            from ..ops import gemm as gemm_ops

            gu = torch.cat([gemm_ops.linear(x, self.w1), gemm_ops.linear(x, self.w3)], dim=-1)
            return gemm_ops.linear(act_ops.glu(gu, "silu"), self.w2.t().contiguous())
        w1, w2, w3 = (w if w.dtype == x.dtype else w.to(x.dtype) for w in (self.w1, self.w2, self.w3))
        return (F.silu(x @ w1.t()) * (x @ w3.t())) @ w2


@dataclass
class MoEConfig:
    # the reference's fields in its order (model/moe.py:1191-1212), this package's additions behind them
    d_model: int = 512
    hidden_size: Optional[int] = None
    num_experts: int = 8
    top_k: int = 2
    bias: bool = False
    z_loss_multiplier: Optional[float] = None
    jitter_eps: Optional[float] = None
    gating_function: GatingFunction = GatingFunction.SOFTMAX
    bias_gamma: Optional[float] = None
    capacity_factor: Optional[float] = None
    shared_expert: bool = False
    ep: Optional["ExpertParallelConfig"] = None      # expert-parallel placement
    fp8_flow_moe: bool = False
    fp8_recipe: str = "none"
    fp8_gemm_threshold: int = 1000000
    adaptive_capacity: bool = False
    adaptive_capacity_target: float = 0.01
    adaptive_capacity_ema: float = 0.3
    routing_replay: bool = False
    extra: dict = field(default_factory=dict)

    def build(self, **kw) -> "MoEBase":
        args = {k: v for k, v in self.__dict__.items() if k != "extra"}
        args.update(kw)
        return MoEBase(**args)


class MoEBase(nn.Module):
    def __init__(self, *, d_model: int, hidden_size: Optional[int] = None, num_experts: int = 8, top_k: int = 2,
                 bias: bool = False, z_loss_multiplier: Optional[float] = None, jitter_eps: Optional[float] = None,
                 gating_function: GatingFunction = GatingFunction.SOFTMAX, bias_gamma: Optional[float] = None,
                 capacity_factor: Optional[float] = None, adaptive_capacity: bool = False,
                 adaptive_capacity_target: float = 0.01, adaptive_capacity_ema: float = 0.3,
                 routing_replay: bool = False, shared_expert: bool = False,
                 ep: Optional[ExpertParallelConfig] = None, fp8_flow_moe: bool = False, fp8_recipe: str = "none",
                 fp8_gemm_threshold: int = 1000000, dtype=None, device=None, init_std: float = 0.01):
        super().__init__()
        self.d_model = d_model
        self.num_experts = num_experts
        self.top_k = top_k
        self.hidden_size = hidden_size or int(8 / 3 * d_model)
        self.hidden_size = ((self.hidden_size + 255) // 256) * 256
        self.capacity_factor = capacity_factor
        self.adaptive_capacity = adaptive_capacity
        self.adaptive_capacity_target = adaptive_capacity_target
        self.adaptive_capacity_ema = adaptive_capacity_ema
        self._adaptive_capacity_ema_drop_rate = 0.0
        self._adaptive_capacity_step = 0
        self._stats: Optional[torch.Tensor] = None  # device [last_dropped, total_dropped, total_routed]
        self._per_expert_drop_counts: Optional[torch.Tensor] = None
        self.router = MoERouter(d_model=d_model, config=MoERouterConfig(
            num_experts=num_experts, top_k=top_k, gating_function=GatingFunction(gating_function),
            routing_replay=routing_replay, bias_init=-1.0, bias_gamma=bias_gamma,
            z_loss_multiplier=z_loss_multiplier, jitter_eps=jitter_eps), device=device)
        self.init_std = init_std
        self.num_local_experts = num_experts
        self.expert_offset = 0
        kw = dict(dtype=dtype, device=device)
        # flattened expert weights, expert e = rows [e*H, (e+1)*H); registered in the reference's order
        # (model/moe.py:1282-1284), which is the order optimizer state is stored in
        self.w1 = nn.Parameter(torch.empty(num_experts * self.hidden_size, d_model, **kw))
        self.w2 = nn.Parameter(torch.empty(num_experts * self.hidden_size, d_model, **kw))
        self.w3 = nn.Parameter(torch.empty(num_experts * self.hidden_size, d_model, **kw))
        self._init_weights()
        self.shared_expert = ExpertMLP(d_model, self.hidden_size, **kw) if shared_expert else None   # reference init
        self.ep = ep or ExpertParallelConfig()
        self._use_grouped_gemm = True
        self.fp8_flow_moe_enabled = fp8_flow_moe
        self.fp8_recipe = fp8_recipe
        self.fp8_gemm_threshold = fp8_gemm_threshold
        self._fp8_flow_moe = None
        self._fused_runtime = None  # ops.moe.FusedMoERuntime once symmetric buffers exist
        self._aux_loss = None
        if fp8_flow_moe:
            self.apply_fp8_flow_moe(True, fp8_recipe, fp8_gemm_threshold)

    def _init_weights(self):
        for w in (self.w1, self.w2, self.w3):
            nn.init.normal_(w, std=self.init_std)

    # -- capacity ---------------------------------------------------------------------------------
    def _capacity(self, num_tokens: int) -> int:
        return int(self.capacity_factor * num_tokens / self.num_experts)

    def _apply_capacity(self, x, weights, indices):
        """Returns ``(x_kept, w_kept, i_kept, dropped, keep_mask)`` (reference: model/moe.py:1395-1448)."""
        T = x.shape[0]
        if self.adaptive_capacity:
            self._update_adaptive_capacity(T, indices)
        capacity = self._capacity(T)
        onehot = torch.zeros(T, self.num_experts, dtype=torch.bool, device=x.device)
        onehot.scatter_(1, indices, True)
        pos = onehot.long().cumsum(0) - 1
        keep_mask = ~(onehot & (pos >= capacity)).any(dim=1)
        per_e = (onehot.sum(0) - capacity).clamp_min(0)
        self._per_expert_drop_counts = per_e
        dropped = T - keep_mask.sum()
        self._record_drops(dropped, T, x.device)
        return x[keep_mask], weights[keep_mask], indices[keep_mask], dropped, keep_mask

    def _record_drops(self, dropped, T, device):
        if self._stats is None or self._stats.device != device:
            self._stats = torch.zeros(3, dtype=torch.long, device=device)
        d = dropped if torch.is_tensor(dropped) else torch.tensor(dropped, device=device)
        self._stats[0] = d
        self._stats[1] += d
        self._stats[2] += T

    def _update_adaptive_capacity(self, num_tokens: int, indices: torch.Tensor):
        if self.capacity_factor is None:
            return
        cf = self.capacity_factor
        onehot = torch.zeros(num_tokens, self.num_experts, dtype=torch.bool, device=indices.device)
        onehot.scatter_(1, indices, True)
        per_e = onehot.sum(0)
        capacity = int(cf * num_tokens / self.num_experts)
        est = float((per_e - capacity).clamp_min(0).sum().item())
        rate = est / max(1, num_tokens)
        a = self.adaptive_capacity_ema
        self._adaptive_capacity_ema_drop_rate = a * rate + (1 - a) * self._adaptive_capacity_ema_drop_rate
        self._adaptive_capacity_step += 1
        if self._adaptive_capacity_ema_drop_rate > self.adaptive_capacity_target * 1.5:
            cf *= 1.1
        elif self._adaptive_capacity_ema_drop_rate < self.adaptive_capacity_target * 0.5:
            cf *= 0.95
        self.capacity_factor = max(1.0, min(4.0, cf))

    # -- expert compute ---------------------------------------------------------------------------
    def _expert_weights(self, e_local: int):
        H = self.hidden_size
        sl = slice(e_local * H, (e_local + 1) * H)
        return self.w1[sl], self.w2[sl], self.w3[sl]

    def _compute_experts_grouped_gemm(self, x, weights, indices):
        """Rows are sorted by local expert: per-expert ``(silu(x w1^T) * (x w3^T)) w2`` on each segment."""
        n_local = self.num_local_experts
        if x.shape[0] == 0:
            return x.new_zeros((0, self.d_model))
        counts = torch.bincount(indices, minlength=n_local).tolist()
        outs, start = [], 0
        for e, c in enumerate(counts):
            if c == 0:
                continue
            seg = x[start:start + c]
            w1, w2, w3 = self._expert_weights(e)
            h = F.silu(seg @ w1.t().to(seg.dtype)) * (seg @ w3.t().to(seg.dtype))
            outs.append(h @ w2.to(seg.dtype))
            start += c
        return torch.cat(outs, dim=0) if outs else x.new_zeros((0, self.d_model))

    _compute_experts_padded_bmm = _compute_experts_grouped_gemm

    # -- phase API (reference: model/moe.py:1602-1714) ----------------------------------------------
    def route(self, x: torch.Tensor):
        """(B,S,D) -> (x_flat, w_flat, i_flat, aux_loss, dropped, keep_mask) after capacity."""
        D = x.shape[-1]
        x_flat = x.reshape(-1, D)
        w, idx, aux = self.router(x)
        w_flat, i_flat = w.reshape(-1, self.top_k), idx.reshape(-1, self.top_k)
        dropped, keep_mask = 0, None
        if self.capacity_factor is not None:
            x_flat, w_flat, i_flat, dropped, keep_mask = self._apply_capacity(x_flat, w_flat, i_flat)
        else:
            self._record_drops(0, x_flat.shape[0], x.device)
        self._aux_loss = aux
        return x_flat, w_flat, i_flat, aux, dropped, keep_mask

    # parameter names as in the reference (model/moe.py), so that keyword calls written against it keep working
    def dispatch(self, x_flat, indices_flat, weights_flat):
        return self.ep.dispatch(x_flat, indices_flat, weights_flat, self.num_experts)

    def local_compute(self, local_x, local_weights, local_indices):
        if self._fp8_flow_moe is not None and local_x.shape[0] > 0:
            return self._fp8_flow_moe(local_x, None, local_indices, 0, self.num_local_experts)
        return self._compute_experts_grouped_gemm(local_x, local_weights, local_indices)

    def combine(self, expert_output, combine_metadata, x_flat, weights_flat, indices_flat):
        out = self.ep.combine(expert_output, combine_metadata, x_flat, weights_flat, indices_flat)
        if self.shared_expert is not None:
            out = out + self.shared_expert(x_flat)
        return out

    def reassemble(self, output, *, dropped, keep_mask, B, S, D):
        if keep_mask is not None:
            full = output.new_zeros((B * S, D))
            full[keep_mask] = output
            output = full
        return output.view(B, S, D)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        B, S, D = x.shape
        if self._can_fuse(x):
            from ..ops import moe as moe_ops

            return moe_ops.fused_moe_forward(self, x)
        x_flat, w_flat, i_flat, aux, dropped, keep_mask = self.route(x)
        local_x, local_w, local_i, meta = self.dispatch(x_flat, i_flat, w_flat)
        expert_out = self.local_compute(local_x, local_w, local_i)
        out = self.combine(expert_out, meta, x_flat, w_flat, i_flat)
        return self.reassemble(out, dropped=dropped, keep_mask=keep_mask, B=B, S=S, D=D)

    def _can_fuse(self, x) -> bool:
        rt = self._fused_runtime
        f = self._fp8_flow_moe
        if f is not None and self.fp8_recipe == "mxfp8" and rt is not None and \
                f.use_fp8(x.numel() // x.shape[-1] * self.top_k / max(self.num_experts, 1)):
            return False  # the MXFP8 expert GEMMs live in the modular path (FP8FlowMoECompute)
        if rt is not None and self.adaptive_capacity:
            # the symmetric receive regions are sized for one capacity; a capacity factor that moves needs the
            # modular path (say so once instead of silently running the slow path)
            if not getattr(self, "_warned_adaptive", False):
                import warnings

                warnings.warn("MoEBase: adaptive_capacity is on, the fused expert-parallel kernels are bypassed "
                              "(their receive buffers are sized for a fixed capacity factor)")
                self._warned_adaptive = True
            return False
        return (rt is not None and _lib.on(x) and x.dtype == torch.bfloat16 and self.w1.dtype == torch.bfloat16
                and self.router.config.normalize_expert_weights is None
                and not (self.router.routing_replay and self.router._replay_mask is not None))

    # -- parallel / fp8 hooks -------------------------------------------------------------------------
    def apply_ep(self, ep: ExpertParallelConfig):
        """Shard the expert weights over the EP group: rank r keeps experts [r*E/ep, (r+1)*E/ep)."""
        self.ep = ep
        if ep.ep_size <= 1:
            return
        assert self.num_experts % ep.ep_size == 0, "num_experts must divide ep_size"
        lo, hi = ep.local_experts(self.num_experts)
        H = self.hidden_size
        with torch.no_grad():
            for name in ("w1", "w3", "w2"):
                w = getattr(self, name)
                setattr(self, name, nn.Parameter(w.data[lo * H:hi * H].clone()))
        self.num_local_experts = hi - lo
        self.expert_offset = lo
        for p in (self.w1, self.w2, self.w3):
            p._ep_sharded = True  # gradients of expert shards are not averaged over the EP group
        if getattr(self.router, "_sp_group", None) is not None:
            self.mark_rows_sharded(self.router._sp_group)     # the shards are new parameter objects: mark them again

    def mark_rows_sharded(self, group) -> None:
        """Sequence-parallel tensor parallelism hands this layer 1 / tp of the rows on every TP rank, and a MoE layer
        is not tensor-parallel: every weight of it then sees a partial gradient that has to be summed over ``group``.
        Gradients may be written by kernels straight into the parameter arena, past any autograd hook, so the arena
        sums the regions of parameters carrying ``_sp_reduce_group``; without an arena the tensor hook does it (per
        backward pass, before accumulation). The router also takes its load statistics over the group."""
        self.router._sp_group = group

        def hook_for(param):
            def fn(g):
                if hasattr(param, "main_grad"):
                    return g
                g = g.contiguous().clone()
                dist.all_reduce(g, group=group)
                return g
            return fn

        for p in self.parameters():
            if getattr(p, "_tp_partial", False) or getattr(p, "_sp_reduce_group", None) is not None:
                continue
            p._sp_reduce_group = group
            p.register_hook(hook_for(p))

    def apply_fp8_flow_moe(self, fp8_flow_moe: bool = True, fp8_recipe: str = "flow_moe",
                           fp8_gemm_threshold: Optional[int] = None):
        enabled = fp8_flow_moe
        self.fp8_flow_moe_enabled = enabled
        self.fp8_recipe = fp8_recipe
        if fp8_gemm_threshold is not None:
            self.fp8_gemm_threshold = fp8_gemm_threshold
        if not enabled or fp8_recipe == "none":
            self._fp8_flow_moe = None
            return
        from ..fp8.flow_moe import FP8FlowMoECompute, FP8FlowMoEConfig
        from ..fp8.recipes import FP8RecipeConfig, FP8RecipeType

        cfg = FP8FlowMoEConfig(enabled=True, fp8_recipe=FP8RecipeConfig(enabled=True,
                                                                        recipe_type=FP8RecipeType(fp8_recipe)))
        self._fp8_flow_moe = FP8FlowMoECompute(cfg, self.d_model, self.hidden_size, self.num_local_experts,
                                               fp8_gemm_threshold=self.fp8_gemm_threshold)
        self._fp8_flow_moe.set_weights(self.w1, self.w2, self.w3)

    # -- observability ---------------------------------------------------------------------------------
    @property
    def aux_loss(self) -> Optional[torch.Tensor]:
        return self._aux_loss

    def _stat(self, i: int) -> int:
        return 0 if self._stats is None else int(self._stats[i].item())

    @property
    def last_dropped(self) -> int:
        return self._stat(0)

    @property
    def last_dropped_slots(self) -> int:
        """Sum of the per-expert overflows of the last forward: the figure the reference reports as ``last_dropped``
        (a token is counted once per over-full expert it chose, so the figure can exceed the token count)."""
        c = self._per_expert_drop_counts
        return 0 if c is None else int(c.sum().item())

    @property
    def total_dropped(self) -> int:
        return self._stat(1)

    @property
    def total_tokens_routed(self) -> int:
        return self._stat(2)

    @property
    def drop_rate(self) -> float:
        t = self.total_tokens_routed
        return 0.0 if t == 0 else self.total_dropped / t

    @property
    def per_expert_drops(self) -> Optional[torch.Tensor]:
        return self._per_expert_drop_counts

    @property
    def adaptive_drop_rate_ema(self) -> float:
        return self._adaptive_capacity_ema_drop_rate

    def reset_drop_stats(self):
        self._stats = None
        self._per_expert_drop_counts = None
        self._adaptive_capacity_ema_drop_rate = 0.0
        self._adaptive_capacity_step = 0

    def get_drop_stats(self) -> dict:
        return {
            "last_dropped": self.last_dropped, "total_dropped": self.total_dropped,
            "total_tokens_routed": self.total_tokens_routed, "drop_rate": self.drop_rate,
            "per_expert_drops": (self._per_expert_drop_counts.tolist()
                                 if self._per_expert_drop_counts is not None else None),
            "capacity_factor": self.capacity_factor, "adaptive_capacity_enabled": self.adaptive_capacity,
            "adaptive_drop_rate_ema": self._adaptive_capacity_ema_drop_rate,
            "adaptive_capacity_step": self._adaptive_capacity_step,
        }
