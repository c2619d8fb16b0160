"""Cross-entropy over bf16 logits without an fp32 copy of the logits.

Forward kernel: one pass for the row log-sum-exp and the picked logit; backward kernel: writes
``(softmax - onehot) * grad / count`` in bf16 (csrc/elementwise.cu ``xent_fwd/bwd``).
Reference: ``F.cross_entropy(logits, labels, ignore_index=-100)`` at model/transformer.py:451-458.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib


class _Xent(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, labels, ignore_index):
        rows, V = logits.shape
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
        lse = torch.empty(rows, device=logits.device, dtype=torch.float32)
        _lib.call("xent_fwd", logits, labels, loss, lse, rows, V, _lib.LL(logits.stride(0)), _lib.LL(ignore_index))
        count = (labels != ignore_index).sum().clamp_min(1).float()
        inv = (1.0 / count).reshape(1)
        ctx.save_for_backward(logits, labels, lse, inv)
        ctx.ignore_index = ignore_index
        return loss.sum() * inv[0]

    @staticmethod
    def backward(ctx, g):
        logits, labels, lse, inv = ctx.saved_tensors
        rows, V = logits.shape
        dlogits = torch.empty_like(logits)
        gs = g.reshape(1).float().contiguous()
        _lib.call("xent_bwd", logits, labels, lse, gs, inv, dlogits, rows, V, _lib.LL(logits.stride(0)),
                  _lib.LL(ctx.ignore_index))
        return dlogits, None, None


def cross_entropy(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100) -> torch.Tensor:
    """Mean token cross-entropy of ``logits [rows, V]`` against ``labels [rows]``."""
    if _lib.on(logits) and logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        return _Xent.apply(logits, labels.contiguous().long(), ignore_index)
    return F.cross_entropy(logits.float(), labels.long(), ignore_index=ignore_index)
