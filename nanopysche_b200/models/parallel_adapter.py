"""Generic parallel hooks for arbitrary ``nn.Module`` models (reference: model/parallel_adapter.py).

A custom-factory model only has to expose ``forward(input_ids, labels=...) -> {"loss": ...}``;
``ensure_parallel_hooks`` binds whichever ``apply_*`` methods it lacks: Megatron-style TP over the
Linear children of each layer (column-wise on all but the last, row-wise + all-reduce on the last),
CP on any ``Attention`` found, EP on any ``MoEBase`` found, FSDP over the layer stack, PP by
trimming the layer stack.
"""
from __future__ import annotations

import types
from typing import Optional

import torch
import torch.nn as nn

from .protocol import PARALLEL_HOOKS, has_hook
from .tp_utils import copy_to_tp_region, differentiable_all_reduce

# attribute names a generic model may use (reference: model/parallel_adapter.py:26-28)
LAYER_STACK_ATTRS = ("blocks", "layers", "layer", "h")
EMBED_ATTRS = ("embeddings", "embed", "wte", "token_embedding")
HEAD_ATTRS = ("lm_head", "head", "output", "proj")
_LAYER_NAMES, _EMBED_NAMES, _HEAD_NAMES = LAYER_STACK_ATTRS, EMBED_ATTRS, HEAD_ATTRS


def find_layer_stack(model: nn.Module):
    """``(attribute name, container)`` of the model's repeated layers, ``None`` when it has none (reference:
    model/parallel_adapter.py:31-38)."""
    for n in LAYER_STACK_ATTRS:
        m = getattr(model, n, None)
        if isinstance(m, (nn.ModuleList, nn.ModuleDict, nn.Sequential)) and len(m) > 0:
            return n, m
    return None


def _layer_stack(model: nn.Module):
    """``find_layer_stack`` for unpacking: ``(None, None)`` when there is no stack."""
    return find_layer_stack(model) or (None, None)


def find_embeddings(model: nn.Module):
    for n in _EMBED_NAMES:
        m = getattr(model, n, None)
        if isinstance(m, nn.Embedding):
            return n, m
    return None, None


def find_head(model: nn.Module):
    for n in _HEAD_NAMES:
        m = getattr(model, n, None)
        if isinstance(m, nn.Linear):
            return n, m
    return None, None


def _layers(stack):
    """Layers of a stack in execution order (a ``ModuleDict`` keyed by layer index is ordered numerically, so
    ``"10"`` follows ``"9"``)."""
    if isinstance(stack, nn.ModuleDict):
        keys = sorted(stack.keys(), key=lambda k: (0, int(k)) if str(k).isdigit() else (1, str(k)))
        return [stack[k] for k in keys]
    return list(stack)


def layer_count(model: nn.Module) -> int:
    """Number of layers in the model's layer stack, 0 when none is found (reference: model/parallel_adapter.py:41-45)."""
    _, stack = _layer_stack(model)
    return len(stack) if stack is not None else 0


def iter_layers(model: nn.Module):
    """The model's layers in execution order (reference: model/parallel_adapter.py:48-57)."""
    _, stack = _layer_stack(model)
    return iter(_layers(stack)) if stack is not None else iter(())


class _RowParallelLinear(nn.Module):
    def __init__(self, lin: nn.Linear, group, tp: int, rank: int):
        super().__init__()
        n = lin.in_features // tp
        self.weight = nn.Parameter(lin.weight.data[:, rank * n:(rank + 1) * n].clone())
        self.weight._tp_sharded = group
        self.bias = lin.bias
        self.group, self.tp, self.rank, self.n = group, tp, rank, n

    def forward(self, x):
        if x.shape[-1] != self.n:  # full-width input: take this rank's slice
            x = x[..., self.rank * self.n:(self.rank + 1) * self.n]
        y = torch.nn.functional.linear(x, self.weight)
        y = differentiable_all_reduce(y, self.group, self.tp)
        return y if self.bias is None else y + self.bias


class _ColParallelLinear(nn.Module):
    def __init__(self, lin: nn.Linear, group, tp: int, rank: int):
        super().__init__()
        n = lin.out_features // tp
        self.weight = nn.Parameter(lin.weight.data[rank * n:(rank + 1) * n].clone())
        self.bias = None if lin.bias is None else nn.Parameter(lin.bias.data[rank * n:(rank + 1) * n].clone())
        self.weight._tp_sharded = group
        if self.bias is not None:
            self.bias._tp_sharded = group
        self.group, self.tp = group, tp

    def forward(self, x):
        x = copy_to_tp_region(x, self.group, self.tp)
        return torch.nn.functional.linear(x, self.weight, self.bias)


def apply_generic_tp(model: nn.Module, tp_mesh, **_):
    """Column-parallel on every Linear child of a layer except the last, row-parallel on the last."""
    import torch.distributed as dist

    group = tp_mesh.get_group() if hasattr(tp_mesh, "get_group") else tp_mesh
    tp, rank = dist.get_world_size(group), dist.get_rank(group)
    _, stack = _layer_stack(model)
    if stack is None or tp <= 1:
        return model
    for layer in _layers(stack):
        if has_hook(layer, "apply_tp"):
            layer.apply_tp(tp_mesh)
            continue
        lins = [(n, m) for n, m in layer.named_children() if isinstance(m, nn.Linear)]
        if len(lins) < 2:
            continue
        for i, (n, m) in enumerate(lins):
            if i < len(lins) - 1:
                if m.out_features % tp == 0:
                    setattr(layer, n, _ColParallelLinear(m, group, tp, rank))
            elif m.in_features % tp == 0:
                setattr(layer, n, _RowParallelLinear(m, group, tp, rank))
    return model


def apply_generic_cp(model: nn.Module, cp_mesh, *, ring=None, uly=None, **_):
    from .attention import Attention

    for m in model.modules():
        if isinstance(m, Attention):
            m.apply_cp(cp_mesh, ring=ring, uly=uly)
    return model


def apply_generic_pp(model: nn.Module, pp_mesh, *, num_stages: Optional[int] = None,
                     stage_idx: Optional[int] = None, **_):
    import torch.distributed as dist

    from ..parallel.pipeline_runtime import stage_layer_ranges

    group = pp_mesh.get_group() if hasattr(pp_mesh, "get_group") else pp_mesh
    num_stages = num_stages or dist.get_world_size(group)
    stage_idx = dist.get_rank(group) if stage_idx is None else stage_idx
    name, stack = _layer_stack(model)
    if stack is None:
        return model
    layers = _layers(stack)
    lo, hi = stage_layer_ranges(len(layers), num_stages)[stage_idx]
    if isinstance(stack, nn.ModuleDict):
        for i, k in enumerate(list(stack.keys())):
            if not (lo <= i < hi):
                del stack[k]
    else:
        setattr(model, name, type(stack)(layers[lo:hi]))
    model._pp_stage = (stage_idx, num_stages)
    return model


def apply_generic_ep(model: nn.Module, ep_config, **_):
    import torch.distributed as dist

    from .moe import ExpertParallelConfig, MoEBase

    if not isinstance(ep_config, ExpertParallelConfig):
        group = ep_config.get_group() if hasattr(ep_config, "get_group") else ep_config
        ep_config = ExpertParallelConfig(ep_size=dist.get_world_size(group), ep_group=group)
    for m in model.modules():
        if isinstance(m, MoEBase):
            m.apply_ep(ExpertParallelConfig(ep_size=ep_config.ep_size, ep_group=ep_config.ep_group,
                                            dispatcher=ep_config.dispatcher))
    return model


def apply_generic_fsdp(model: nn.Module, dp_mesh=None, *, param_dtype=None, reduce_dtype=torch.float32, **kw):
    from ..parallel.fsdp import MixedPrecision, shard_module

    mp = MixedPrecision(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    _, stack = _layer_stack(model)
    if stack is not None:
        for layer in _layers(stack):
            shard_module(layer, dp_mesh, mp_policy=mp)
    shard_module(model, dp_mesh, mp_policy=mp)
    return model


def apply_generic_compile(model: nn.Module, **_):
    return model


def init_generic_weights(model: nn.Module, device=None, world_mesh=None, std: float = 0.02):
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, std)
    return model


_GENERIC = {"apply_tp": apply_generic_tp, "apply_cp": apply_generic_cp, "apply_pp": apply_generic_pp,
            "apply_ep": apply_generic_ep, "apply_fsdp": apply_generic_fsdp, "apply_compile": apply_generic_compile,
            "init_weights": init_generic_weights}


def missing_parallel_hooks(model: nn.Module) -> list[str]:
    return [h for h in PARALLEL_HOOKS if not has_hook(model, h)]


def ensure_parallel_hooks(model: nn.Module) -> nn.Module:
    """Bind generic ``apply_*`` methods for every hook the model lacks (no-op for built-in models)."""
    for name in missing_parallel_hooks(model):
        fn = _GENERIC[name]
        setattr(model, name, types.MethodType(lambda self, *a, _fn=fn, **k: _fn(self, *a, **k), model))
    return model
