"""Embedding lookup whose backward adds straight into the fp32 gradient arena.

Forward is the plain gather. Backward: when the weight carries a ``main_grad`` view of the arena (``optim/arena.py``)
and the incoming gradient is bf16 on CUDA, one kernel does ``main_grad[ids[t]] += dy[t]`` with 16-byte vector
reductions (``csrc/elementwise.cu::embedding_bwd_kernel``) instead of building a dense ``[V, D]`` bf16 gradient by
sort + segment sum and copying it into the arena. Elsewhere the dense gradient is formed with ``index_add_``.

The reference uses ``nn.Embedding`` (model/transformer.py of the reference, token embedding of ``Transformer``).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids)
        ctx.weight = weight
        return F.embedding(ids, weight)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        w = ctx.weight
        D = w.shape[1]
        dy2 = dy.reshape(-1, D)
        # a weight whose gradient is partial per tensor-parallel rank goes through autograd so that its reduce hook runs
        mg = None if getattr(w, "_tp_partial", False) else getattr(w, "main_grad", None)
        if mg is not None and _lib.on(dy2) and dy2.dtype == torch.bfloat16 and mg.dtype == torch.float32 and D % 4 == 0 \
                and ids.dtype == torch.int64:
            dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
            flat = ids.reshape(-1)
            flat = flat if flat.is_contiguous() else flat.contiguous()
            first = not getattr(w, "_main_grad_dirty", False)
            _lib.call("embedding_bwd", dy2, flat, mg, _lib.LL(flat.numel()), D, _lib.LL(w.shape[0]), int(first))
            w._main_grad_dirty = True
            cb = getattr(w, "_grad_ready_cb", None)   # the arena's overlapped gradient reduction
            if cb is not None:
                cb(w)
            return None, None
        g = torch.zeros(w.shape, device=dy2.device, dtype=torch.float32)
        g.index_add_(0, ids.reshape(-1), dy2.float())
        return None, g.to(w.dtype)


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``weight[ids]``; see the module docstring for the backward."""
    if weight.requires_grad and torch.is_grad_enabled():
        return _Embedding.apply(ids, weight)
    return F.embedding(ids, weight)
