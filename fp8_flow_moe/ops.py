"""FP8-Flow-MoE operators: blockwise e4m3 (de)quantisation, scaling-aware transpose, fused
SwiGLU+quantise, permute+pad / unpermute+unpad, and the block-scaled grouped GEMM.

Every operator has a pure-PyTorch implementation (the CPU path and the oracle). On a CUDA device
with the in-tree sm_100a library present, the quantisation / transpose / SwiGLU-quantise operators
run as hand-written kernels (``csrc/quant.cu``).

Scales are fp32 ``amax / 448`` per block (``mxfp8``: rounded up to a power of two), stored
``[rows, cols / block]`` for 1xB activation blocks and ``[rows / 128, cols / 128]`` for weights.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

FP8_BLOCK_SIZE = 128
FP8_MAX = 448.0
FP8_DTYPE = torch.float8_e4m3fn


def _kernels():
    """The ctypes kernel library if a GPU and the library are available, else None."""
    import os

    if not torch.cuda.is_available() or os.environ.get("FP8_FLOW_MOE_NO_NATIVE", "0") == "1":
        return None
    from ._native import native

    try:
        return native()
    except Exception as e:  # noqa: BLE001
        # on a GPU box the kernels are the product: say why they are missing instead of quietly running ATen ops
        raise RuntimeError(f"fp8_flow_moe: a GPU is present but the kernel library could not be loaded or built ({e}); "
                           "run `python -m fp8_flow_moe.build`, or set FP8_FLOW_MOE_NO_NATIVE=1 for the PyTorch "
                           "path") from e


def _pow2_ceil(s: torch.Tensor) -> torch.Tensor:
    return torch.exp2(torch.ceil(torch.log2(s.clamp_min(1e-30))))


def quantize_to_fp8(x: torch.Tensor, block_size: int = FP8_BLOCK_SIZE, pow2_scales: bool = False
                    ) -> Tuple[torch.Tensor, torch.Tensor]:
    """1 x ``block_size`` blockwise quantisation along the last dim -> (e4m3 tensor, fp32 scales)."""
    cols = x.shape[-1]
    assert cols % block_size == 0, "last dim must be a multiple of the block size"
    k = _kernels()
    if k is not None and x.is_cuda and x.dtype == torch.bfloat16 and block_size == 128 and not pow2_scales \
            and x.is_contiguous():
        return k.quant_1x128(x)
    xb = x.float().reshape(*x.shape[:-1], cols // block_size, block_size)
    scale = xb.abs().amax(dim=-1).clamp_min(1e-12) / FP8_MAX
    if pow2_scales:
        scale = _pow2_ceil(scale)
    q = (xb / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)
    return q.reshape(x.shape), scale


def dequantize_from_fp8(q: torch.Tensor, scales: torch.Tensor, block_size: Optional[int] = None,
                        dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    cols = q.shape[-1]
    if scales.dim() == q.dim() and scales.shape[:-1] == q.shape[:-1]:
        block = block_size or cols // scales.shape[-1]
        k = _kernels()
        if k is not None and q.is_cuda and block == 128 and dtype == torch.bfloat16 and q.is_contiguous():
            return k.dequant_1x128(q, scales)
        qb = q.float().reshape(*q.shape[:-1], cols // block, block)
        return (qb * scales.unsqueeze(-1)).reshape(q.shape).to(dtype)
    # 128x128 weight blocks
    br, bc = q.shape[-2] // scales.shape[-2], q.shape[-1] // scales.shape[-1]
    s = scales.repeat_interleave(br, dim=-2).repeat_interleave(bc, dim=-1)
    return (q.float() * s).to(dtype)


def quantize_weight_blockwise(w: torch.Tensor, block: int = FP8_BLOCK_SIZE) -> Tuple[torch.Tensor, torch.Tensor]:
    """``block x block`` weight quantisation -> (e4m3 [R, C], fp32 scales [R/block, C/block])."""
    R, C = w.shape[-2:]
    assert R % block == 0 and C % block == 0
    k = _kernels()
    if k is not None and w.is_cuda and w.dtype == torch.bfloat16 and block == 128 and w.dim() == 2 and \
            w.is_contiguous():
        return k.quant_128x128(w)
    wb = w.float().reshape(*w.shape[:-2], R // block, block, C // block, block)
    scale = wb.abs().amax(dim=(-3, -1)).clamp_min(1e-12) / FP8_MAX
    q = (wb / scale[..., :, None, :, None]).clamp(-FP8_MAX, FP8_MAX).to(FP8_DTYPE)
    return q.reshape(w.shape), scale


def scaling_aware_transpose(q: torch.Tensor, scales: torch.Tensor, block_size: int = FP8_BLOCK_SIZE
                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Transpose a 1xB-quantised ``[M, N]`` tensor into a 1xB-quantised ``[N, M]`` one without going
    through bf16 in memory: each (B x B) tile is rescaled from its B row scales to one column-block
    scale per output row. Needed by wgrad, whose contraction runs over the token axis."""
    M, N = q.shape
    assert M % block_size == 0 and N % block_size == 0
    k = _kernels()
    if k is not None and q.is_cuda and block_size == 128 and q.is_contiguous():
        return k.transpose_1x128(q, scales)
    deq = dequantize_from_fp8(q, scales, block_size, dtype=torch.float32)
    return quantize_to_fp8(deq.t().contiguous(), block_size)


def fused_silu_multiply_quantize(gate: torch.Tensor, up: torch.Tensor, block_size: int = FP8_BLOCK_SIZE
                                 ) -> Tuple[torch.Tensor, torch.Tensor]:
    """``quantize(silu(gate) * up)`` in one pass."""
    k = _kernels()
    if k is not None and gate.is_cuda and gate.dtype == torch.bfloat16 and block_size == 128 and gate.dim() == 2 \
            and gate.stride(1) == 1 and up.stride(1) == 1 and gate.shape[1] % 128 == 0:
        return k.swiglu_quant(gate, up)  # row-strided views (halves of a [gate | up] buffer) are fine
    return quantize_to_fp8((F.silu(gate.float()) * up.float()).to(gate.dtype), block_size)


def fused_swiglu_quantize(gate_up: torch.Tensor, block_size: int = FP8_BLOCK_SIZE):
    """Same for a fused ``[gate | up]`` tensor."""
    g, u = gate_up.chunk(2, dim=-1)
    if gate_up.is_cuda and gate_up.dim() == 2:
        return fused_silu_multiply_quantize(g, u, block_size)
    return fused_silu_multiply_quantize(g.contiguous(), u.contiguous(), block_size)


class _ScatterRows(torch.autograd.Function):
    """``out[row_map[i]] = x[i]`` into ``total`` zero rows (kernel); backward gathers."""

    @staticmethod
    def forward(ctx, x, row_map, total):
        ctx.save_for_backward(row_map)
        out = x.new_zeros((total, x.shape[1]))
        return _kernels().move_rows(x, out, row_map, None, scatter=True)

    @staticmethod
    def backward(ctx, g):
        (row_map,) = ctx.saved_tensors
        g = g if g.is_contiguous() else g.contiguous()
        dx = torch.empty((row_map.numel(), g.shape[1]), device=g.device, dtype=g.dtype)
        return _kernels().move_rows(g, dx, row_map, None, scatter=False), None, None


class _GatherRows(torch.autograd.Function):
    """``out[i] = y[row_map[i]] * w[i]`` (kernel); backward scatters ``g * w`` and reduces ``<g, y>`` per row."""

    @staticmethod
    def forward(ctx, y, row_map, weights):
        ctx.save_for_backward(y, row_map, weights if weights is not None else y.new_empty(0))
        ctx.has_w = weights is not None
        out = torch.empty((row_map.numel(), y.shape[1]), device=y.device, dtype=y.dtype)
        return _kernels().move_rows(y, out, row_map, weights, scatter=False)

    @staticmethod
    def backward(ctx, g):
        y, row_map, w = ctx.saved_tensors
        g = g if g.is_contiguous() else g.contiguous()
        gw = g * w.reshape(-1, 1).to(g.dtype) if ctx.has_w else g
        dy = _kernels().move_rows(gw.contiguous(), y.new_zeros(y.shape), row_map, None, scatter=True)
        dw = (g.float() * y[row_map].float()).sum(-1).reshape(w.shape).to(w.dtype) if ctx.has_w and \
            ctx.needs_input_grad[2] else None
        return dy, None, dw


def fused_permute_pad(x: torch.Tensor, indices: torch.Tensor, num_experts: int, pad_multiple: int = FP8_BLOCK_SIZE
                      ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sort rows by expert and pad every expert segment to a multiple of ``pad_multiple``.

    ``x [n, D]``, ``indices [n]`` -> ``(permuted [P, D] with zero padding rows, row_map [n] position of
    each input row in the permuted tensor, tokens_per_expert [E] padded segment sizes)``.
    """
    n = x.shape[0]
    k = _kernels()
    if k is not None and x.is_cuda and n > 0 and x.is_contiguous() and (x.shape[1] * x.element_size()) % 16 == 0:
        # counting-sort positions and the row scatter as kernels (no argsort); the output size depends on the data,
        # so one scalar comes back to the host
        row_map, padded = k.expert_rank(indices, num_experts, pad_multiple)
        return _ScatterRows.apply(x, row_map, int(padded.sum().item())), row_map, padded
    order = torch.argsort(indices, stable=True)
    counts = torch.bincount(indices, minlength=num_experts)
    padded = (counts + pad_multiple - 1) // pad_multiple * pad_multiple
    starts = torch.cumsum(padded, 0) - padded
    seg_start = torch.cumsum(counts, 0) - counts
    sorted_e = indices[order]
    pos_sorted = starts[sorted_e] + (torch.arange(n, device=x.device) - seg_start[sorted_e])
    row_map = torch.empty(n, dtype=torch.long, device=x.device)
    row_map[order] = pos_sorted
    total = int(padded.sum().item())
    out = x.new_zeros((total, x.shape[1]))
    out[row_map] = x
    return out, row_map, padded


def fused_unpermute_unpad(y: torch.Tensor, row_map: torch.Tensor, weights: Optional[torch.Tensor] = None
                          ) -> torch.Tensor:
    """Inverse of ``fused_permute_pad``: gather the original rows (optionally times a per-row weight)."""
    k = _kernels()
    if k is not None and y.is_cuda and y.is_contiguous() and (y.shape[1] * y.element_size()) % 16 == 0 and \
            row_map.numel() > 0 and (weights is None or y.dtype == torch.bfloat16):
        return _GatherRows.apply(y, row_map.to(torch.int64).contiguous(), weights)
    out = y[row_map]
    return out if weights is None else out * weights.reshape(-1, 1).to(out.dtype)


def fp8_grouped_gemm(xq: torch.Tensor, x_scales: torch.Tensor, wq: torch.Tensor, w_scales: torch.Tensor,
                     tokens_per_expert: torch.Tensor, out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    """``y[rows of e] = dequant(x[rows of e]) @ dequant(w[e]).T`` for consecutive expert segments.

    ``xq [P, K]`` e4m3 with 1x128 scales ``[P, K/128]``; ``wq [E, N, K]`` e4m3 with 128x128 scales
    ``[E, N/128, K/128]``; ``tokens_per_expert [E]`` segment sizes (padded)."""
    E, N, K = wq.shape
    out = torch.zeros((xq.shape[0], N), device=xq.device, dtype=out_dtype)
    start = 0
    for e, c in enumerate(tokens_per_expert.tolist()):
        if c:
            xs = dequantize_from_fp8(xq[start:start + c], x_scales[start:start + c], dtype=torch.float32)
            we = dequantize_from_fp8(wq[e], w_scales[e], dtype=torch.float32)
            out[start:start + c] = (xs @ we.t()).to(out_dtype)
        start += c
    return out
