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
                     lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8, weight_decay: float = 0.1,
                     max_grad_norm: Optional[float] = 1.0, fused_moe: bool = True):
    """Returns ``(optimizer, arena | None)``. ``dp_group``: ranks holding replicas of the non-expert
    parameters (their gradients are averaged); ``ep_group``: ranks the experts are spread over."""
    p0 = next(model.parameters())
    if p0.device.type != "cuda":
        opt = torch.optim.AdamW(model.parameters(), lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        return opt, None
    if dp_group is None and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and \
            getattr(model, "_needs_grad_sync", False):
        dp_group = dist.group.WORLD
    arena = ParamArena(model, dp_group=dp_group, device=p0.device)
    moes = moe_layers(model)
    if moes and fused_moe and tokens_per_rank:
        from .ops.moe import build_runtime

        grp = ep_group if ep_group is not None else moes[0].ep.ep_group
        build_runtime(moes, tokens=tokens_per_rank, group=grp if moes[0].ep.ep_size > 1 else None, device=p0.device)
    opt = ArenaAdamW(arena, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, max_grad_norm=max_grad_norm)
    return opt, arena
