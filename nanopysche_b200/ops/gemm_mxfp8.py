"""MXFP8 GEMM op (csrc/gemm_mxfp8_sm100.cu) with its PyTorch reference.

MXFP8: e4m3 values with one shared power-of-two scale (an e8m0 exponent byte, value ``2^(b - 127)``) per block of
32 consecutive elements along the contraction dimension. ``mx_quantize(x)`` returns ``(q, sf)`` with ``q`` the e4m3
tensor ``[rows, K]`` and ``sf`` the exponent bytes in the chunk layout the tensor core reads (``sf_index``);
``gemm_mxfp8(aq, sfa, bq, sfb)`` computes ``dequant(a) @ dequant(b)^T`` with the scaling done by the block-scaled
tcgen05 MMA. With ``mblk_group`` (one group id per 128-row block of ``aq``) block ``i`` uses rows
``[g * rows_per_group, (g + 1) * rows_per_group)`` of ``bq``: the grouped (per-expert) form.

Stands where the reference's ``mxfp8`` recipe hands linears to torchao's MX tensors (cli.py:28-186, fp8 recipe
flag; fp8/recipes.py of the reference).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib

SF_CHUNK = 512  # bytes: 128 rows x 4 blocks of 32


def sf_index(rows: int, K: int, device=None) -> torch.Tensor:
    """Byte offset of the scale of (row r, 32-block j) in the chunked buffer, as an int64 ``[rows, K/32]`` tensor:
    chunk ``(r // 128) * (K // 128) + j // 4``, inside it ``(r % 32) * 16 + ((r % 128) // 32) * 4 + j % 4``."""
    r = torch.arange(rows, device=device).view(-1, 1)
    j = torch.arange(K // 32, device=device).view(1, -1)
    chunk = (r // 128) * (K // 128) + j // 4
    return chunk * SF_CHUNK + (r % 32) * 16 + ((r % 128) // 32) * 4 + (j % 4)


def sf_bytes(rows: int, K: int) -> int:
    return ((rows + 127) // 128) * (K // 128) * SF_CHUNK


def mx_quantize_ref(x: torch.Tensor):
    """PyTorch statement of the quantiser: per 1x32 block ``e = ceil(log2(amax / 448))`` clamped to [-127, 127]."""
    rows, K = x.shape
    xf = x.float().view(rows, K // 32, 32)
    am = xf.abs().amax(-1)
    mant, ex = torch.frexp(am / 448.0)
    e = torch.where(mant == 0.5, ex - 1, ex)
    e = torch.where(am > 0, e, torch.full_like(e, -127)).clamp(-127, 127)
    q = (xf * torch.exp2(-e.float()).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(rows, K)
    sf = torch.full((sf_bytes(rows, K),), 127, dtype=torch.uint8, device=x.device)
    sf[sf_index(rows, K, x.device).reshape(-1)] = (e + 127).to(torch.uint8).reshape(-1)
    return q, sf


def mx_quantize(x: torch.Tensor):
    """bf16 ``[rows, K]`` (K a multiple of 128, unit column stride) -> ``(e4m3 [rows, K], uint8 scale chunks)``."""
    if not x.is_cuda:
        return mx_quantize_ref(x)
    rows, K = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and K % 128 == 0
    q = torch.empty((rows, K), device=x.device, dtype=torch.float8_e4m3fn)
    sf = torch.full((sf_bytes(rows, K),), 127, dtype=torch.uint8, device=x.device)
    _lib.check(_lib.lib().np_mx_quant(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)), C.c_void_p(q.data_ptr()),
                                      C.c_longlong(K), C.c_void_p(sf.data_ptr()), rows, K,
                                      C.c_void_p(_lib.stream())), "mx_quant")
    return q, sf


def mx_dequantize_bf16(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    """e4m3 ``[rows, K]`` + chunked exponent bytes -> bf16 (one kernel on CUDA)."""
    rows, K = q.shape
    if not q.is_cuda:
        return mx_dequantize(q, sf).to(torch.bfloat16)
    assert q.stride(1) == 1 and K % 128 == 0
    out = torch.empty((rows, K), device=q.device, dtype=torch.bfloat16)
    _lib.check(_lib.lib().np_mx_dequant(C.c_void_p(q.data_ptr()), C.c_longlong(q.stride(0)), C.c_void_p(sf.data_ptr()),
                                        C.c_void_p(out.data_ptr()), C.c_longlong(K), rows, K,
                                        C.c_void_p(_lib.stream())), "mx_dequant")
    return out


# ------------------------------------------------------------------------------------ 128-wide power-of-two blocks
def _pow2_exp(am: torch.Tensor) -> torch.Tensor:
    mant, ex = torch.frexp(am / 448.0)
    e = torch.where(mant == 0.5, ex - 1, ex)
    return torch.where(am > 0, e, torch.full_like(e, -127)).clamp(-127, 127)


def flow_quantize_act_ref(x: torch.Tensor, swiglu: bool = False):
    """PyTorch statement of ``flow_quantize_act``: one power-of-two scale per 1x128 block, stored as four equal
    exponent bytes (the four 1x32 hardware blocks it spans)."""
    xf = x.float()
    if swiglu:
        g, u = xf.chunk(2, dim=-1)
        xf = torch.nn.functional.silu(g) * u
    rows, K = xf.shape
    xb = xf.view(rows, K // 128, 128)
    e = _pow2_exp(xb.abs().amax(-1))
    q = (xb * torch.exp2(-e.float()).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(rows, K)
    sf = torch.zeros((sf_bytes(rows, K),), dtype=torch.uint8, device=x.device)
    sf[sf_index(rows, K, x.device).reshape(-1)] = (e + 127).to(torch.uint8).repeat_interleave(4, dim=1).reshape(-1)
    return q, sf


def flow_quantize_act(x: torch.Tensor, swiglu: bool = False, out=None, h_out: Optional[torch.Tensor] = None):
    """bf16 ``[rows, K]`` -> ``(e4m3 [rows, K], exponent chunks)`` with 1x128 power-of-two scales (FP8-Flow-MoE
    activations in the form the block-scaled tensor-core MMA consumes). ``swiglu``: ``x`` is ``[rows, 2K]`` =
    ``[gate | up]`` and ``silu(gate) * up`` is what gets quantised (the reference's ``fused_swiglu_quantize``);
    ``h_out`` (bf16 ``[rows, K]``) then also receives the unquantised product."""
    if not x.is_cuda:
        q, sf = flow_quantize_act_ref(x, swiglu)
        if h_out is not None:
            g, u = x.float().chunk(2, dim=-1)
            h_out.copy_((torch.nn.functional.silu(g) * u).to(h_out.dtype))
        return q, sf
    rows = x.shape[0]
    K = x.shape[1] // 2 if swiglu else x.shape[1]
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and K % 128 == 0
    if out is None:
        q = torch.empty((rows, K), device=x.device, dtype=torch.float8_e4m3fn)
        sf = torch.zeros((sf_bytes(rows, K),), dtype=torch.uint8, device=x.device)
    else:
        q, sf = out
    _lib.check(_lib.lib().np_flow_quant_act(C.c_void_p(x.data_ptr()), C.c_longlong(x.stride(0)),
                                            C.c_void_p(q.data_ptr()), C.c_longlong(q.stride(0)),
                                            C.c_void_p(sf.data_ptr()), rows, K, int(swiglu),
                                            C.c_void_p(h_out.data_ptr() if h_out is not None else 0),
                                            C.c_longlong(h_out.stride(0) if h_out is not None else 0),
                                            C.c_void_p(_lib.stream())), "flow_quant_act")
    return q, sf


def flow_quantize_weight_ref(w: torch.Tensor, experts: int = 1, transpose: bool = False):
    R, Cc = w.shape[0] // experts, w.shape[1]
    wf = w.float().view(experts, R, Cc)
    if transpose:
        wf = wf.transpose(1, 2).contiguous()
        R, Cc = Cc, R
    blk = wf.view(experts, R // 128, 128, Cc // 128, 128)
    e = _pow2_exp(blk.abs().amax(dim=(2, 4)))                                   # [E, R/128, C/128]
    q = (blk * torch.exp2(-e.float())[:, :, None, :, None]).clamp(-448, 448).to(torch.float8_e4m3fn)
    q = q.view(experts * R, Cc)
    sf = (e + 127).to(torch.uint8).reshape(-1, 1).expand(-1, SF_CHUNK).reshape(-1).contiguous()
    return q, sf


def flow_quantize_weight(w: torch.Tensor, experts: int = 1, transpose: bool = False, out=None, out_rows: int = 0,
                         out_row0: int = 0):
    """``experts`` stacked ``[R, C]`` bf16 matrices -> e4m3 with one power-of-two scale per 128x128 block
    (FP8-Flow-MoE weights); ``transpose`` writes every matrix as ``[C, R]`` so that a GEMM can contract over R.
    With ``out=(q, sf)``, ``out_rows`` and ``out_row0`` expert ``e`` is written to rows ``e * out_rows + out_row0`` of a
    larger output (several weights stacked per expert)."""
    if not w.is_cuda:
        assert out is None
        return flow_quantize_weight_ref(w, experts, transpose)
    assert w.dtype == torch.bfloat16 and w.is_contiguous() and w.shape[0] % experts == 0
    R, Cc = w.shape[0] // experts, w.shape[1]
    assert R % 128 == 0 and Cc % 128 == 0
    oshape = (experts * Cc, R) if transpose else (experts * R, Cc)
    if out is None:
        q = torch.empty(oshape, device=w.device, dtype=torch.float8_e4m3fn)
        sf = torch.empty((sf_bytes(oshape[0], oshape[1]),), dtype=torch.uint8, device=w.device)
    else:
        q, sf = out
    _lib.check(_lib.lib().np_flow_quant_weight(C.c_void_p(w.data_ptr()), C.c_void_p(q.data_ptr()),
                                               C.c_void_p(sf.data_ptr()), experts, R, Cc, int(transpose),
                                               int(out_rows), int(out_row0), C.c_void_p(_lib.stream())),
               "flow_quant_weight")
    return q, sf


def mx_dequantize(q: torch.Tensor, sf: torch.Tensor) -> torch.Tensor:
    rows, K = q.shape
    e = sf[sf_index(rows, K, q.device).reshape(-1)].view(rows, K // 32).float() - 127.0
    return (q.float().view(rows, K // 32, 32) * torch.exp2(e).unsqueeze(-1)).view(rows, K)


def gemm_mxfp8_ref(aq, sfa, bq, sfb, mblk_group=None, rows_per_group: int = 0, out_dtype=torch.bfloat16):
    a, b = mx_dequantize(aq, sfa), mx_dequantize(bq, sfb)
    if mblk_group is None:
        return (a @ b.t()).to(out_dtype)
    N = rows_per_group
    out = torch.zeros((a.shape[0], N), device=aq.device, dtype=torch.float32)
    for i, g in enumerate(mblk_group.tolist()):
        if g >= 0:
            out[i * 128:(i + 1) * 128] = a[i * 128:(i + 1) * 128] @ b[g * N:(g + 1) * N].t()
    return out.to(out_dtype)


def gemm_mxfp8(aq: torch.Tensor, sfa: torch.Tensor, bq: torch.Tensor, sfb: torch.Tensor, *,
               out: Optional[torch.Tensor] = None, out_dtype: torch.dtype = torch.bfloat16,
               mblk_group: Optional[torch.Tensor] = None, mblk_rows: Optional[torch.Tensor] = None,
               rows_per_group: int = 0, fill: Optional[dict] = None) -> torch.Tensor:
    """``fill``: extra ``MxGemmArgs`` fields (arrival-flag wait, per-row destination table and completion counters of
    the fused expert-parallel path; with ``row_dst`` the output goes to peer buffers and ``out`` may be None)."""
    if not aq.is_cuda:
        return gemm_mxfp8_ref(aq, sfa, bq, sfb, mblk_group, rows_per_group, out_dtype)
    M, K = aq.shape
    N = rows_per_group if mblk_group is not None else bq.shape[0]
    assert K % 128 == 0 and N % 128 == 0 and bq.shape[0] % 128 == 0 and aq.stride(1) == 1 and bq.stride(1) == 1
    assert sfa.numel() >= sf_bytes(M, K) and sfb.numel() >= sf_bytes(bq.shape[0], K)
    push = bool(fill and fill.get("row_dst"))
    if out is None and not push:
        out = torch.empty((M, N), device=aq.device, dtype=out_dtype)
    a = _lib.MxGemmArgs()
    a.A, a.B, a.sfa, a.sfb = aq.data_ptr(), bq.data_ptr(), sfa.data_ptr(), sfb.data_ptr()
    a.C = out.data_ptr() if out is not None else None
    a.lda, a.ldb, a.ldc = aq.stride(0), bq.stride(0), (out.stride(0) if out is not None else N)
    a.a_rows, a.b_rows = aq.shape[0], bq.shape[0]
    a.M, a.N, a.K = M, N, K
    a.out_f32 = int(out is not None and out.dtype == torch.float32)
    if mblk_group is not None:
        a.mode, a.mblk_group, a.group_stride_b = 1, mblk_group.data_ptr(), rows_per_group
        a.mblk_rows = mblk_rows.data_ptr() if mblk_rows is not None else None
    for k, v in (fill or {}).items():
        setattr(a, k, v)
    _lib.check(_lib.lib().np_gemm_mxfp8(C.byref(a), C.c_void_p(_lib.stream())), "gemm_mxfp8")
    return out


class _MXLinear(torch.autograd.Function):
    """Forward through the MXFP8 GEMM (activations and weight quantised per 1x32 block along the contraction);
    both backward GEMMs in bf16 on the unquantised tensors."""

    @staticmethod
    def forward(ctx, x, w):
        from .gemm import gemm

        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        xq, sx = mx_quantize(x2)
        wq, sw = mx_quantize(w if w.is_contiguous() else w.contiguous())
        y = gemm_mxfp8(xq, sx, wq, sw)
        ctx.save_for_backward(x2, w)
        ctx.x_shape = x.shape
        ctx.gemm = gemm
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from .gemm import _wgrad_into

        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        dx = ctx.gemm(dy2, w, b_mn=True).view(ctx.x_shape) if ctx.needs_input_grad[0] else None
        dw = _wgrad_into(w, dy2, x2) if (ctx.needs_input_grad[1] or hasattr(w, "main_grad")) else None
        return dx, dw


def mx_linear_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 2 and
            w.shape[1] % 128 == 0 and w.shape[0] % 128 == 0)


def mx_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w.T (+ bias)`` with the forward GEMM in MXFP8."""
    y = _MXLinear.apply(x, w)
    return y if bias is None else y + bias


class _MXExpertMLP(torch.autograd.Function):
    """``(silu(x w1_e^T) * (x w3_e^T)) w2_e`` over rows grouped per expert in multiples of 128: the three forward
    GEMMs in MXFP8 (grouped form), the backward GEMMs in bf16 per expert on the unquantised tensors."""

    @staticmethod
    def forward(ctx, xp, w1, w3, w2, counts, quantised):
        w1q, s1, w3q, s3, w2q, s2 = quantised
        E = len(counts)
        H, D = w1.shape[0] // E, w1.shape[1]
        blocks = xp.shape[0] // 128
        grp = torch.repeat_interleave(torch.arange(E, device=xp.device, dtype=torch.int32),
                                      torch.tensor([c // 128 for c in counts], device=xp.device),
                                      output_size=blocks)
        xb = xp.to(torch.bfloat16)
        xq, sx = mx_quantize(xb)
        g = gemm_mxfp8(xq, sx, w1q, s1, mblk_group=grp, rows_per_group=H)
        u = gemm_mxfp8(xq, sx, w3q, s3, mblk_group=grp, rows_per_group=H)
        h = (torch.nn.functional.silu(g.float()) * u.float()).to(torch.bfloat16)
        hq, sh = mx_quantize(h)
        y = gemm_mxfp8(hq, sh, w2q, s2, mblk_group=grp, rows_per_group=D, out_dtype=xp.dtype)
        ctx.save_for_backward(xb, g, u, w1, w3, w2)
        ctx.counts, ctx.x_dtype = counts, xp.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        from .gemm import gemm

        xb, g, u, w1, w3, w2 = ctx.saved_tensors
        counts = ctx.counts
        E = len(counts)
        H, D = w1.shape[0] // E, w1.shape[1]
        dyb = dy.to(torch.bfloat16)
        dyb = dyb if dyb.is_contiguous() else dyb.contiguous()
        dx = torch.zeros_like(xb)
        dw1, dw3, dw2 = (torch.zeros(w.shape, device=w.device, dtype=torch.bfloat16) for w in (w1, w3, w2))
        wb = [w.detach().to(torch.bfloat16) for w in (w1, w3, w2)]
        start = 0
        for e, c in enumerate(counts):
            if c:
                r = slice(start, start + c)
                we1, we3, we2 = (w[e * H:(e + 1) * H] for w in wb)
                gf, uf = g[r].float(), u[r].float()
                sg = torch.sigmoid(gf)
                dh = gemm(dyb[r], we2).float()                                   # [c, H] = dy w2_e^T
                he = (gf * sg * uf).to(torch.bfloat16)
                dg = (dh * uf * (sg * (1 + gf * (1 - sg)))).to(torch.bfloat16)
                du = (dh * gf * sg).to(torch.bfloat16)
                dx[r] = gemm(dg, we1, b_mn=True) + gemm(du, we3, b_mn=True)     # [c, D]
                dw2[e * H:(e + 1) * H] = gemm(he, dyb[r], a_mn=True, b_mn=True)  # [H, D] = h^T dy
                dw1[e * H:(e + 1) * H] = gemm(dg, xb[r], a_mn=True, b_mn=True)
                dw3[e * H:(e + 1) * H] = gemm(du, xb[r], a_mn=True, b_mn=True)
            start += c
        return dx.to(ctx.x_dtype), dw1.to(w1.dtype), dw3.to(w3.dtype), dw2.to(w2.dtype), None, None


def mx_expert_mlp(xp: torch.Tensor, w1: torch.Tensor, w3: torch.Tensor, w2: torch.Tensor, counts, quantised):
    """Expert MLP over ``xp [P, D]`` whose rows are grouped per expert (``counts``: rows per expert, multiples of
    128); ``w1, w3, w2: [E*H, D]``; ``quantised``: the six tensors of ``mx_quantize`` on w1, w3 and on w2 transposed
    per expert to ``[E*D, H]``."""
    return _MXExpertMLP.apply(xp, w1, w3, w2, list(counts), tuple(quantised))
