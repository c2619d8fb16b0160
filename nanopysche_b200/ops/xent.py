"""Cross-entropy over bf16 logits without an fp32 copy of the logits.

Forward kernel: one pass for the row log-sum-exp and the picked logit; backward kernel: writes
``(softmax - onehot) * grad / count`` in bf16 (csrc/elementwise.cu ``xent_fwd/bwd``).
Reference: ``F.cross_entropy(logits, labels, ignore_index=-100)`` at model/transformer.py:451-458.

``linear_cross_entropy`` is the head projection and the loss together, in chunks of rows: the ``[rows, V]`` logits of
one chunk live only until its loss (forward) or its gradient (backward, which recomputes them) has been taken, so
neither the logits nor their gradient exist for the whole batch (at 4096 x 32000 in bf16 they are 262 MB each).
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


def _rows_fwd(logits: torch.Tensor, labels: torch.Tensor, ignore_index: int):
    """Per-row loss (0 for ignored rows) and log-sum-exp of one chunk of logits."""
    rows, V = logits.shape
    if _lib.on(logits) and logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        loss = torch.empty(rows, device=logits.device, dtype=torch.float32)
        lse = torch.empty(rows, device=logits.device, dtype=torch.float32)
        _lib.call("xent_fwd", logits, labels, loss, lse, rows, V, _lib.LL(logits.stride(0)), _lib.LL(ignore_index))
        return loss, lse
    lf = logits.float()
    lse = torch.logsumexp(lf, dim=-1)
    keep = labels != ignore_index
    picked = lf.gather(1, labels.clamp_min(0).unsqueeze(1)).squeeze(1)
    return torch.where(keep, lse - picked, torch.zeros_like(lse)), lse


def _rows_bwd(logits: torch.Tensor, labels: torch.Tensor, lse: torch.Tensor, gs: torch.Tensor, inv: torch.Tensor,
              ignore_index: int) -> torch.Tensor:
    """``(softmax - onehot) * gs * inv`` for one chunk (zero rows where the label is ignored), in the logits' dtype."""
    rows, V = logits.shape
    if _lib.on(logits) and logits.dtype == torch.bfloat16 and logits.stride(1) == 1 and logits.stride(0) % 8 == 0:
        dlogits = torch.empty_like(logits)
        _lib.call("xent_bwd", logits, labels, lse, gs, inv, dlogits, rows, V, _lib.LL(logits.stride(0)),
                  _lib.LL(ignore_index))
        return dlogits
    keep = (labels != ignore_index).unsqueeze(1)
    p = torch.exp(logits.float() - lse.unsqueeze(1))
    p.scatter_add_(1, labels.clamp_min(0).unsqueeze(1), -torch.ones(rows, 1, device=logits.device))
    return (p * keep * (gs * inv)).to(logits.dtype)


class _LinearXent(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, labels, ignore_index, chunk):
        from .gemm import gemm

        T = x.shape[0]
        count = (labels != ignore_index).sum().clamp_min(1).float()
        inv = (1.0 / count).reshape(1)
        lse = torch.empty(T, device=x.device, dtype=torch.float32)
        total = torch.zeros((), device=x.device, dtype=torch.float32)
        for s in range(0, T, chunk):
            e = min(s + chunk, T)
            loss_rows, lse_rows = _rows_fwd(gemm(x[s:e], w), labels[s:e], ignore_index)
            lse[s:e] = lse_rows
            total += loss_rows.sum()
        ctx.save_for_backward(x, w, labels, lse, inv)
        ctx.ignore_index, ctx.chunk = ignore_index, chunk
        return total * inv[0]

    @staticmethod
    def backward(ctx, g):
        from .gemm import _wgrad_into, gemm

        x, w, labels, lse, inv = ctx.saved_tensors
        T = x.shape[0]
        gs = g.reshape(1).float().contiguous()
        dx = torch.empty_like(x) if ctx.needs_input_grad[0] else None
        want_dw = ctx.needs_input_grad[1] or hasattr(w, "main_grad")
        dw = None
        for s in range(0, T, ctx.chunk):
            e = min(s + ctx.chunk, T)
            xc = x[s:e]
            dlogits = _rows_bwd(gemm(xc, w), labels[s:e], lse[s:e].contiguous(), gs, inv, ctx.ignore_index)
            if dx is not None:
                dx[s:e] = gemm(dlogits, w, b_mn=True)
            if want_dw:
                part = _wgrad_into(w, dlogits, xc)       # into the gradient arena when the weight lives there
                if part is not None:
                    dw = part if dw is None else dw + part
        return dx, dw, None, None, None


def linear_cross_entropy(x: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, ignore_index: int = -100,
                         chunk_rows: int = 1024) -> torch.Tensor:
    """Mean token cross-entropy of ``x [rows, D] @ w [V, D]^T`` against ``labels [rows]`` without ever holding the
    logits of more than ``chunk_rows`` rows; the backward pass recomputes each chunk's logits (one more head GEMM per
    step). Same value and gradients as ``cross_entropy(linear(x, w), labels)``."""
    x2 = x if x.is_contiguous() else x.contiguous()
    if x2.dtype != w.dtype:
        x2 = x2.to(w.dtype)
    return _LinearXent.apply(x2, w, labels.contiguous().long(), ignore_index, max(int(chunk_rows), 1))
