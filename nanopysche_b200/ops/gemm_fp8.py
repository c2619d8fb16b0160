"""Block-scaled fp8 GEMM op (csrc/gemm_fp8_sm100.cu) with its PyTorch reference.

``gemm_fp8_block(aq, sa, bq, sb)`` computes ``dequant(aq, sa) @ dequant(bq, sb)^T`` where ``aq [M, K]`` is
e4m3 with 1x128 scales ``sa [M, K/128]`` and ``bq [N, K]`` is e4m3 with 128x128 scales ``sb [N/128, K/128]``.
With ``mblk_group`` (one group id per 128-row block of ``aq``) the B operand of block ``i`` is rows
``[g*rows_per_group, ...)`` of ``bq`` - the grouped (per-expert) form.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib


def gemm_fp8_block_ref(aq, sa, bq, sb, mblk_group=None, rows_per_group: int = 0, out_dtype=torch.bfloat16):
    M, K = aq.shape
    a = aq.float().view(M, K // 128, 128) * sa.view(M, K // 128, 1)
    Nb = bq.shape[0]
    b = bq.float().view(Nb // 128, 128, K // 128, 128) * sb.view(Nb // 128, 1, K // 128, 1)
    b = b.view(Nb, K)
    a = a.view(M, K)
    if mblk_group is None:
        return (a @ b.t()).to(out_dtype)
    N = rows_per_group
    out = torch.zeros((M, N), device=aq.device, dtype=torch.float32)
    for i, g in enumerate(mblk_group.tolist()):
        if g >= 0:
            out[i * 128:(i + 1) * 128] = a[i * 128:(i + 1) * 128] @ b[g * N:(g + 1) * N].t()
    return out.to(out_dtype)


def gemm_fp8_block(aq: torch.Tensor, sa: torch.Tensor, bq: torch.Tensor, sb: torch.Tensor, *,
                   out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
                   mblk_group: Optional[torch.Tensor] = None, mblk_rows: Optional[torch.Tensor] = None,
                   rows_per_group: int = 0, fill: Optional[dict] = None) -> torch.Tensor:
    """See the module docstring. ``fill`` lets callers set the flag-wait / peer-push fields of the
    argument block (used by the fused MoE layer)."""
    if not aq.is_cuda:
        return gemm_fp8_block_ref(aq, sa, bq, sb, mblk_group, rows_per_group, out_dtype)
    M, K = aq.shape
    N = rows_per_group if mblk_group is not None else bq.shape[0]
    assert K % 128 == 0 and N % 128 == 0 and aq.stride(1) == 1 and bq.stride(1) == 1
    assert sa.dtype == torch.float32 and sb.dtype == torch.float32 and sa.is_contiguous() and sb.is_contiguous()
    push = fill is not None and fill.get("row_dst")
    if out is None and not push:
        out = torch.empty((M, N), device=aq.device, dtype=out_dtype)
    a = _lib.Fp8GemmArgs()
    a.A, a.B, a.sa, a.sb = aq.data_ptr(), bq.data_ptr(), sa.data_ptr(), sb.data_ptr()
    a.lda, a.ldb = aq.stride(0), bq.stride(0)
    a.a_rows, a.b_rows = aq.shape[0], bq.shape[0]
    a.M, a.N, a.K = M, N, K
    if out is not None:
        a.C, a.ldc, a.out_f32 = out.data_ptr(), out.stride(0), int(out.dtype == torch.float32)
    else:
        a.ldc = N
    if mblk_group is not None:
        a.mode, a.mblk_group, a.group_stride_b = 1, mblk_group.data_ptr(), rows_per_group
        a.mblk_rows = mblk_rows.data_ptr() if mblk_rows is not None else None
    for k, v in (fill or {}).items():
        setattr(a, k, v)
    _lib.check(_lib.lib().np_gemm_fp8_block(C.byref(a), C.c_void_p(_lib.stream())), "gemm_fp8_block")
    return out


class _Fp8BlockLinear(torch.autograd.Function):
    """Forward GEMM on e4m3 operands (1x128 activation scales, 128x128 weight scales); backward GEMMs in bf16."""

    @staticmethod
    def forward(ctx, x, w):
        from fp8_flow_moe import ops as fops

        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        xq, xs = fops.quantize_to_fp8(x2)
        wq, ws = fops.quantize_weight_blockwise(w if w.is_contiguous() else w.contiguous())
        y = gemm_fp8_block(xq, xs.contiguous(), wq, ws.contiguous())
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .gemm import _wgrad_into, gemm

        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = gemm(dy2, w, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _wgrad_into(w, dy2, x2) if (ctx.needs_input_grad[1] or hasattr(w, "main_grad")) else None
        return dx, dw


def fp8_block_linear_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2 and
            w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0)


def fp8_block_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    y = _Fp8BlockLinear.apply(x, w)
    return y if bias is None else y + bias
