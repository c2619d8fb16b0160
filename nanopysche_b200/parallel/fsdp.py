"""Data-parallel sharding and activation checkpointing (reference: distributed/fsdp.py:30-133).

Two sharding back ends sit behind the reference's hook names:

* ``shard_module`` / ``apply_generic_fsdp``: per-module FSDP (ZeRO-3) through PyTorch's
  ``fully_shard`` with the reference's mixed-precision policy. It is the plain-collective baseline
  and what runs on CPU/gloo.
* the flat parameter arena (``optim/arena.py``) shards optimizer state and gradients over the
  data-parallel group (ZeRO-2 layout) and runs reduce-scatter + AdamW + all-gather as one sm_100a
  kernel over peer memory (``ops/zero.py``); ``parallelize_model`` picks it on CUDA.
* ``fully_shard_linears`` (``backend="sharded"``) additionally shards the bf16 weights of the linear layers by rows
  (ZeRO-3 layout): the all-gather of a weight runs inside the GEMM that consumes it and the weight gradient comes
  back reduce-scattered (``ops/fsdp_fused.py``); everything that is not such a weight stays with the arena's ZeRO
  step.
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
    # "auto" | "torch" (fully_shard) | "arena" (flat ZeRO arena, CUDA) | "sharded" (arena + row-sharded linear
    # weights gathered inside their GEMMs, CUDA)
    backend: str = "auto"


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

    def __init__(self, module: nn.Module, use_reentrant: bool = False):
        super().__init__()
        self.module = module
        self.use_reentrant = use_reentrant

    def forward(self, *args, **kwargs):
        return checkpoint(self.module, *args, use_reentrant=self.use_reentrant, **kwargs)

    def __getattr__(self, name):  # hooks (apply_tp, feed_forward, ...) resolve on the wrapped module
        try:
            return super().__getattr__(name)
        except AttributeError:
            return getattr(super().__getattr__("module"), name)


def apply_activation_checkpointing(model: nn.Module, mode: str = "full", block_interval: Optional[int] = None):
    """``full``: every block; ``selected_blocks``: every ``block_interval``-th block."""
    from ..models.parallel_adapter import find_layer_stack

    _, stack = find_layer_stack(model) or (None, None)
    if stack is None or mode in (None, "none"):
        return model
    keys = list(stack.keys()) if isinstance(stack, nn.ModuleDict) else list(range(len(stack)))
    for n, k in enumerate(keys):
        if mode == "selected_blocks" and block_interval and n % block_interval != 0:
            continue
        if not isinstance(stack[k], ActivationCheckpointing):
            stack[k] = ActivationCheckpointing(stack[k])
    return model


def apply_generic_fsdp(model: nn.Module, dp_mesh=None, dp_config: Optional[DataParallelConfig] = None, *,
                       param_dtype: Optional[torch.dtype] = None, reduce_dtype: Optional[torch.dtype] = None):
    """``param_dtype`` / ``reduce_dtype`` (the reference's keywords, distributed/fsdp.py) override the config's."""
    cfg = dp_config or DataParallelConfig()
    if param_dtype is not None or reduce_dtype is not None:
        import dataclasses as _dc

        cfg = _dc.replace(cfg, **({"param_dtype": param_dtype} if param_dtype is not None else {}),
                          **({"reduce_dtype": reduce_dtype} if reduce_dtype is not None else {}))
    return shard_module(model, dp_mesh, mp_policy=MixedPrecision(cfg.param_dtype, cfg.reduce_dtype))


def fully_shard_linears(model: nn.Module, group, *, device=None, skip=()):
    """Shard the weight of every eligible ``nn.Linear`` by rows over ``group`` (ZeRO-3 layout for the GEMM weights).

    Eligible: bf16 CUDA weight without bias, not tied to an embedding, rows divisible into shards of a multiple of
    128 rows. ``lin.weight`` becomes this rank's ``[rows / n, in]`` shard, tagged with the shared ``FSDPRuntime``
    (``_fsdp_rt``) so ``ops.gemm.linear`` runs it as all-gather-inside-GEMM with a reduce-scattered weight
    gradient, and with ``_ep_sharded`` so the parameter arena treats it as rank-local (no second gradient
    reduction; its squared norm is summed over the ranks). Returns the runtime, or ``None`` when nothing qualified.

    Plays the role of ``fully_shard`` on the transformer blocks (reference: distributed/fsdp.py:18-83)."""
    import torch.distributed as dist

    from ..ops.fsdp_fused import FSDPRuntime

    n = dist.get_world_size(group)
    if n <= 1:
        return None
    rank = dist.get_rank(group)
    tied = {id(m.weight) for m in model.modules() if isinstance(m, nn.Embedding)}
    todo = []
    for name, m in model.named_modules():
        if not isinstance(m, nn.Linear) or m.bias is not None or name in skip:
            continue
        w = m.weight
        if id(w) in tied or not w.is_cuda or w.dtype != torch.bfloat16 or getattr(w, "_ep_sharded", False):
            continue
        if not FSDPRuntime.supported(w.shape[0], n) or w.shape[1] % 64:
            continue
        todo.append((name, m))
    if not todo:
        return None
    rt = FSDPRuntime(group, max(m.weight.numel() for _, m in todo), device=device or todo[0][1].weight.device)
    for name, m in todo:
        full = m.weight.data
        ns = full.shape[0] // n
        shard = nn.Parameter(full[rank * ns:(rank + 1) * ns].clone())
        shard._fsdp_rt = rt
        shard._fsdp_full_rows = full.shape[0]
        shard._ep_sharded = True
        m.weight = shard
    model._fsdp_linear_runtime = rt
    model._fsdp_sharded_linears = [name for name, _ in todo]
    return rt


def gather_sharded_linears(model: nn.Module) -> dict:
    """``{module name: full bf16 weight}`` of the linears sharded by ``fully_shard_linears`` (NCCL all-gather; for
    checkpoints and evaluation outside the sharded path)."""
    import torch.distributed as dist

    rt = getattr(model, "_fsdp_linear_runtime", None)
    out = {}
    if rt is None:
        return out
    mods = dict(model.named_modules())
    for name in model._fsdp_sharded_linears:
        w = mods[name].weight.data
        full = torch.empty((w.shape[0] * rt.n, w.shape[1]), device=w.device, dtype=w.dtype)
        dist.all_gather_into_tensor(full, w.contiguous(), group=rt.group)
        out[name] = full
    return out
