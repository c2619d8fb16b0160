"""B200 training engine glue: turns a parallelised model into the fused execution form.

``prepare_training`` (1) moves parameters into the flat arena (fused QKV / gate-up weights, fp32
``main_grad`` buffers written directly by the wgrad GEMMs), (2) builds the symmetric-memory runtime
for the MoE layers so dispatch / expert GEMMs / combine run as fused kernels over peer memory and
(3) returns the arena optimizer. On CPU it returns a plain AdamW so the same call works everywhere.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .models.moe import MoEBase
from .optim.arena import ArenaAdamW, ParamArena


def moe_layers(model: nn.Module) -> list:
    return [m for m in model.modules() if isinstance(m, MoEBase)]


def prepare_training(model: nn.Module, *, tokens_per_rank: Optional[int] = None, dp_group=None, ep_group=None,
                     replicate_group=None,
                     lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1,
                     max_grad_norm: Optional[float] = 1.0, fused_moe: bool = True):
    """Returns ``(optimizer, arena | None)``. ``dp_group``: ranks holding replicas of the non-expert
    parameters (their gradients are averaged; optimizer state is sharded over them); ``ep_group``: ranks the
    experts are spread over; ``replicate_group``: under hybrid sharding (HSDP) the ranks that hold the same
    optimizer shard (``dp_group`` is then the shard group)."""
    p0 = next(model.parameters())
    if dp_group is not None and dist.is_initialized() and dist.get_world_size(dp_group) <= 1:
        dp_group = None
    if p0.device.type != "cuda":
        opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        return opt, None
    if any(type(p).__name__ == "DTensor" for p in model.parameters()):
        # wrapped by torch's FSDP2 (``--fsdp-backend torch``): the parameters are sharded DTensors that the flat arena
        # cannot alias; the library's fused AdamW steps the shards
        opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, fused=True)
        return opt, None
    if dp_group is None and hasattr(model, "_replica_group"):
        dp_group = model._replica_group   # set by parallelize_model: the ranks holding the same parameters (dp x ep x cp)
    elif dp_group is None and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and \
            getattr(model, "_needs_grad_sync", False):
        if getattr(model, "_tp_enabled", False) or getattr(model, "_pp_enabled", False):
            raise ValueError("prepare_training: the model is tensor- or pipeline-parallel; pass dp_group= (the ranks "
                             "that hold replicas of this rank's parameters) - averaging over the whole world would "
                             "mix different shards")
        dp_group = dist.group.WORLD
    if replicate_group is None:
        replicate_group = getattr(model, "_replicate_group", None)   # HSDP: set by parallelize_model
    arena = ParamArena(model, dp_group=dp_group, device=p0.device, replicate_group=replicate_group,
                       expert_replica_group=getattr(model, "_expert_replica_group", None))
    moes = moe_layers(model)
    if moes and fused_moe and tokens_per_rank:
        from .ops.moe import build_runtime

        grp = ep_group if ep_group is not None else moes[0].ep.ep_group
        build_runtime(moes, tokens=tokens_per_rank, group=grp if moes[0].ep.ep_size > 1 else None, device=p0.device)
    opt = ArenaAdamW(arena, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, max_grad_norm=max_grad_norm)
    rt = getattr(moes[0], "_fused_runtime", None) if moes else None
    if rt is not None:
        # ranks outside the expert-parallel group that hold the same layers and route other tokens: copies of the
        # expert shards on other data-parallel ranks (incl. context-parallel peers) and, under sequence-parallel TP,
        # the TP peers. Their load counts belong to the same DeepSeek-V3 bias update.
        rt.extra_count_groups = [g for g in (getattr(model, "_expert_replica_group", None),
                                             getattr(moes[0].router, "_sp_group", None)) if g is not None]
        if rt.score_bias_all is not None:
            opt.post_step_hooks.append(rt.update_router_bias)
        opt.post_step_hooks.append(rt.end_step)
    opt.post_step_hooks.append(_cp_end_step)
    if any(m._fp8_flow_moe is not None for m in moes):
        # the fused AdamW writes the weights from a kernel (no autograd version bump): drop the quantised copies
        def _drop_quantised_weights():
            for m in moes:
                if m._fp8_flow_moe is not None:
                    m._fp8_flow_moe._wq_cache = None

        opt.post_step_hooks.append(_drop_quantised_weights)
    fs = getattr(model, "_fsdp_linear_runtime", None)
    if fs is not None:
        opt.post_step_hooks.append(fs.end_step)
    return opt, arena


def _cp_end_step():
    """Fold the epochs of the fused context-parallel runtimes (created lazily by the attention layers)."""
    from .parallel.context_parallel import _FUSED_RUNTIMES

    for rt in _FUSED_RUNTIMES.values():
        rt.end_step()


class GraphedTrainStep:
    """One training step (forward + backward + clip + AdamW) captured into a CUDA graph.

    The step launches well over a thousand kernels; replaying them as one graph removes the host from
    the critical path. What makes the step capturable: nothing in it synchronises with the host, flag
    epochs and the optimizer schedule are read from device memory (``SymmetricHeap.epoch_base``,
    ``ArenaAdamW._hyper``), gradient synchronisation runs as in-tree kernels over peer memory, and the
    batch is copied into a static input buffer before each replay.

    ``step(ids)`` returns the (device) loss tensor of that step; ``loss_fn(out)`` picks what is
    back-propagated (default ``loss + aux_loss``).
    """

    def __init__(self, model: nn.Module, optimizer: ArenaAdamW, sample_ids: torch.Tensor, warmup: int = 3,
                 loss_fn=None):
        self.model, self.opt = model, optimizer
        self.static_ids = sample_ids.clone()
        self.loss_fn = loss_fn or (lambda out: out["loss"] if out.get("aux_loss") is None
                                   else out["loss"] + out["aux_loss"])
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_loss: Optional[torch.Tensor] = None
        self._warm = warmup

    def _eager(self, hyper_ready: bool):
        out = self.model(self.static_ids, labels=self.static_ids)
        self.loss_fn(out).backward()
        self.opt.step(_hyper_ready=hyper_ready)
        self.opt.zero_grad(set_to_none=True)
        return out["loss"].detach()

    def capture(self):
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(self._warm):
                self._eager(False)
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.opt.update_hyper()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self.static_loss = self._eager(True)
        return self

    def step(self, ids: torch.Tensor) -> torch.Tensor:
        if self.graph is None:
            self.capture()
            # the capture itself does not execute; fall through to a first replay with this batch
        self.static_ids.copy_(ids, non_blocking=True)
        self.opt.update_hyper()
        self.graph.replay()
        return self.static_loss
