"""Tensor-parallel conjugate operators (reference: model/tp_utils.py:25-57).

The reference only has the output-side all-reduce with an identity backward and omits the
input-side operator, so upstream gradients stay partial per TP rank. Both Megatron operators are
provided here: ``copy_to_tp_region`` (forward identity, backward all-reduce) and
``differentiable_all_reduce`` / ``reduce_from_tp_region`` (forward all-reduce, backward identity),
plus the sequence-parallel pair (all-gather <-> reduce-scatter along the sequence dim).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class _AllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        y = x.clone()
        dist.all_reduce(y, op=dist.ReduceOp.SUM, group=group)
        return y

    @staticmethod
    def backward(ctx, g):
        return g, None


class _CopyToRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous().clone()
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=ctx.group)
        return g, None


class _AllGatherSeq(torch.autograd.Function):
    """Forward: all-gather along ``dim``; backward: reduce-scatter."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        n = dist.get_world_size(group)
        xs = x.movedim(dim, 0).contiguous()
        out = torch.empty((n * xs.shape[0], *xs.shape[1:]), device=x.device, dtype=x.dtype)
        dist.all_gather_into_tensor(out, xs, group=group)
        return out.movedim(0, dim)

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        gs = g.movedim(ctx.dim, 0).contiguous()
        out = torch.empty((gs.shape[0] // n, *gs.shape[1:]), device=g.device, dtype=g.dtype)
        _reduce_scatter(out, gs, ctx.group)
        return out.movedim(0, ctx.dim), None, None


class _ReduceScatterSeq(torch.autograd.Function):
    """Forward: reduce-scatter along ``dim``; backward: all-gather."""

    @staticmethod
    def forward(ctx, x, group, dim):
        ctx.group, ctx.dim = group, dim
        n = dist.get_world_size(group)
        xs = x.movedim(dim, 0).contiguous()
        out = torch.empty((xs.shape[0] // n, *xs.shape[1:]), device=x.device, dtype=x.dtype)
        _reduce_scatter(out, xs, group)
        return out.movedim(0, dim)

    @staticmethod
    def backward(ctx, g):
        n = dist.get_world_size(ctx.group)
        gs = g.movedim(ctx.dim, 0).contiguous()
        out = torch.empty((n * gs.shape[0], *gs.shape[1:]), device=g.device, dtype=g.dtype)
        dist.all_gather_into_tensor(out, gs, group=ctx.group)
        return out.movedim(0, ctx.dim), None, None


def _reduce_scatter(out, inp, group):
    if inp.is_cuda:
        dist.reduce_scatter_tensor(out, inp, op=dist.ReduceOp.SUM, group=group)
    else:  # gloo has no reduce_scatter: all-reduce then slice
        tmp = inp.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp[r * out.shape[0]:(r + 1) * out.shape[0]])


def differentiable_all_reduce(tensor: torch.Tensor, group=None, tp_size: int = 1) -> torch.Tensor:
    """Sum over the TP group in forward, identity in backward (no-op when ``tp_size <= 1``)."""
    if tp_size <= 1 or group is None:
        return tensor
    return _AllReduce.apply(tensor, group)


reduce_from_tp_region = differentiable_all_reduce


def copy_to_tp_region(tensor: torch.Tensor, group=None, tp_size: int = 1) -> torch.Tensor:
    """Identity in forward, sum over the TP group in backward."""
    if tp_size <= 1 or group is None:
        return tensor
    return _CopyToRegion.apply(tensor, group)


def gather_seq(tensor, group=None, tp_size: int = 1, dim: int = 1):
    """Sequence-parallel entry: all-gather the sequence shards (backward: reduce-scatter)."""
    if tp_size <= 1 or group is None:
        return tensor
    return _AllGatherSeq.apply(tensor, group, dim)


def scatter_seq(tensor, group=None, tp_size: int = 1, dim: int = 1):
    """Sequence-parallel exit: reduce-scatter along the sequence (backward: all-gather)."""
    if tp_size <= 1 or group is None:
        return tensor
    return _ReduceScatterSeq.apply(tensor, group, dim)
