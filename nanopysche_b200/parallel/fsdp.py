"""Data-parallel sharding and activation checkpointing (reference: distributed/fsdp.py:30-133).

Two sharding back ends sit behind the reference's hook names:

* ``shard_module`` / ``apply_generic_fsdp``: per-module FSDP (ZeRO-3) through PyTorch's
  ``fully_shard`` with the reference's mixed-precision policy. It is the plain-collective baseline
  and what runs on CPU/gloo.
* the flat parameter arena (``optim/arena.py``) shards optimizer state and gradients over the
  data-parallel group (ZeRO-2 layout) and runs reduce-scatter + AdamW + all-gather as one sm_100a
  kernel over peer memory (``ops/zero.py``); ``parallelize_model`` picks it on CUDA.
"""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum
from typing import Optional

import torch
import torch.nn as nn
from torch.utils.checkpoint import checkpoint


class DataParallelType(str, Enum):
    fsdp = "fsdp"
    hsdp = "hsdp"
    ddp = "ddp"


class TransformerDataParallelWrappingStrategy(str, Enum):
    full = "full"
    fine_grained = "fine_grained"


@dataclass
class MixedPrecision:
    param_dtype: Optional[torch.dtype] = None
    reduce_dtype: Optional[torch.dtype] = torch.float32


@dataclass
class DataParallelConfig:
    name: DataParallelType = DataParallelType.fsdp
    param_dtype: Optional[torch.dtype] = None
    reduce_dtype: torch.dtype = torch.float32
    wrapping_strategy: TransformerDataParallelWrappingStrategy = TransformerDataParallelWrappingStrategy.full
    prefetch_factor: int = 0
    backend: str = "auto"  # "auto" | "torch" (fully_shard) | "arena" (flat ZeRO arena, CUDA)


def _mesh_ok(mesh) -> bool:
    try:
        return mesh is not None and mesh.size() > 1
    except Exception:  # noqa: BLE001
        return False


def shard_module(module: nn.Module, dp_mesh=None, *, reshard_after_forward: bool = True,
                 mp_policy: Optional[MixedPrecision] = None):
    """FSDP-wrap one module over ``dp_mesh`` (no-op for a trivial mesh or an already wrapped module)."""
    if not _mesh_ok(dp_mesh) or getattr(module, "_np_sharded", False):
        return module
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    mp = mp_policy or MixedPrecision()
    pol = MixedPrecisionPolicy(param_dtype=mp.param_dtype, reduce_dtype=mp.reduce_dtype)
    fully_shard(module, mesh=dp_mesh, reshard_after_forward=reshard_after_forward, mp_policy=pol)
    module._np_sharded = True
    return module


class ActivationCheckpointing(nn.Module):
    """Recompute the wrapped module in backward (non-reentrant checkpoint)."""

    def __init__(self, module: nn.Module):
        super().__init__()
        self.module = module

    def forward(self, *args, **kwargs):
        return checkpoint(self.module, *args, use_reentrant=False, **kwargs)

    def __getattr__(self, name):  # hooks (apply_tp, feed_forward, ...) resolve on the wrapped module
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("module"), name)


def apply_activation_checkpointing(model: nn.Module, mode: str = "full", block_interval: Optional[int] = None):
    """``full``: every block; ``selected_blocks``: every ``block_interval``-th block."""
    from ..models.parallel_adapter import find_layer_stack

    _, stack = find_layer_stack(model)
    if stack is None or mode in (None, "none"):
        return model
    keys = list(stack.keys()) if isinstance(stack, nn.ModuleDict) else list(range(len(stack)))
    for n, k in enumerate(keys):
        if mode == "selected_blocks" and block_interval and n % block_interval != 0:
            continue
        if not isinstance(stack[k], ActivationCheckpointing):
            stack[k] = ActivationCheckpointing(stack[k])
    return model


def apply_generic_fsdp(model: nn.Module, dp_mesh=None, dp_config: Optional[DataParallelConfig] = None):
    cfg = dp_config or DataParallelConfig()
    return shard_module(model, dp_mesh, mp_policy=MixedPrecision(cfg.param_dtype, cfg.reduce_dtype))
