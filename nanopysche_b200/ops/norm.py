"""RMSNorm op: fused sm_100a kernel (csrc/elementwise.cu) for bf16 CUDA rows, fp32 PyTorch otherwise.

Math of the reference (model/norm.py:38-47): upcast to fp32, ``x * rsqrt(mean(x^2) + eps) * w``,
cast back. The kernel form optionally fuses the residual add in front (``h = x + res``) and returns
``h`` as well, so a block reads and writes the hidden state once per norm.
"""
from __future__ import annotations

import torch

from . import _lib


def rms_norm_ref(x, weight, eps=1e-6, residual=None):
    h = x if residual is None else x + residual
    hf = h.float()
    y = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps)
    y = (y * weight.float()).to(x.dtype)
    return y if residual is None else (y, h)


def _kernel_ok(x, weight):
    return _lib.on(x) and x.dtype == torch.bfloat16 and weight.dtype == torch.float32 and \
        x.shape[-1] % 8 == 0 and x.shape[-1] <= 8192


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, residual, eps):
        D = x.shape[-1]
        x2 = x.reshape(-1, D)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, D)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        h = torch.empty_like(x2) if residual is not None else None
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        _lib.call("rmsnorm_fwd", x2, r2, weight, y, h, rstd, rows, D, float(eps))
        ctx.save_for_backward(h if h is not None else x2, weight, rstd)
        ctx.has_res = residual is not None
        ctx.shape = x.shape
        if residual is not None:
            return y.view(x.shape), h.view(x.shape)
        return y.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dh=None):
        xin, weight, rstd = ctx.saved_tensors
        rows, D = xin.shape
        dy2 = dy.reshape(rows, D)
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dres = None
        if ctx.has_res and dh is not None:
            dres = dh.reshape(rows, D)
            dres = dres if dres.is_contiguous() else dres.contiguous()
        dx = torch.empty_like(xin)
        parts = _lib.lib().np_rmsnorm_bwd_parts(rows)
        scratch = torch.empty((parts, D), device=xin.device, dtype=torch.float32)
        # weights whose gradient is partial per TP rank go through autograd so their reduce hook runs
        mg = None if getattr(weight, "_tp_partial", False) else getattr(weight, "main_grad", None)
        if mg is not None:
            first = not getattr(weight, "_main_grad_dirty", False)
            _lib.call("rmsnorm_bwd", dy2, xin, weight, rstd, dres, dx, mg, scratch, rows, D, int(not first))
            weight._main_grad_dirty = True
            dw = None
        else:
            dw = torch.empty(D, device=xin.device, dtype=torch.float32)
            _lib.call("rmsnorm_bwd", dy2, xin, weight, rstd, dres, dx, dw, scratch, rows, D, 0)
        dx = dx.view(ctx.shape)
        if ctx.has_res:
            return dx, dw, dx, None
        return dx, dw, None, None


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None):
    """``norm(x [+ residual]) * weight``; returns ``(y, x + residual)`` when a residual is given."""
    if _kernel_ok(x, weight) and (residual is None or (residual.dtype == x.dtype and residual.is_cuda)):
        return _RMSNorm.apply(x, weight, residual, eps)
    return rms_norm_ref(x, weight, eps, residual)


def rms_norm_quant(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, residual: torch.Tensor | None = None,
                   return_bf16: bool = False):
    """RMSNorm whose output is already quantised for an fp8 GEMM: ``(q e4m3 [rows, D], scales fp32 [rows, D / 128])``
    with 1x128 blocks and ``scale = amax / 448`` - bit-identical to quantising the bf16 result of ``rms_norm``, in
    one pass over the row. Also returns ``x + residual`` when a residual is given and the bf16 output when
    ``return_bf16``. Forward only (inference, or the recompute half of a checkpointed block)."""
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    if not (_kernel_ok(x, weight) and D % 128 == 0):
        from fp8_flow_moe import ops as fops

        out = rms_norm_ref(x2, weight, eps, None if residual is None else residual.reshape(-1, D))
        y, h = (out if residual is not None else (out, None))
        q, s = fops.quantize_to_fp8(y)
        res = [q, s]
    else:
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        r2 = None
        if residual is not None:
            r2 = residual.reshape(-1, D)
            r2 = r2 if r2.is_contiguous() else r2.contiguous()
        rows = x2.shape[0]
        q = torch.empty((rows, D), device=x.device, dtype=torch.float8_e4m3fn)
        s = torch.empty((rows, D // 128), device=x.device, dtype=torch.float32)
        y = torch.empty_like(x2) if return_bf16 else None
        h = torch.empty_like(x2) if residual is not None else None
        _lib.call("rmsnorm_quant_fwd", x2, r2, weight, y, h, None, q, s, rows, D, float(eps))
        res = [q, s]
    if residual is not None:
        res.append(h.view(x.shape))
    if return_bf16:
        res.append(y.view(x.shape))
    return tuple(res)
