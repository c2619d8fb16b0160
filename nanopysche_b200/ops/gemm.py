"""GEMM ops: the tcgen05 bf16 GEMM (csrc/gemm_sm100.cu) on CUDA tensors, torch.matmul on CPU.

``gemm`` is the raw entry: ``C[M, N] (+)= alpha * sum_k A(m, k) * B(n, k)`` where each operand is
either K-major (``[rows, K]`` row-major, ``*_mn=False``) or MN-major (``[K, rows]`` row-major).
That single contraction covers forward (``x @ w.T``), dgrad (``dy @ w``: B MN-major) and wgrad
(``dy.T @ x``: both MN-major) without materialising a transpose.

``linear`` is the autograd function used by the model layers in place of ``nn.functional.linear``
(reference: model/attention.py:141-143,189; model/feed_forward.py:75). When the weight carries a
``main_grad`` buffer (the flat fp32 gradient arena of ``optim.arena``), the wgrad GEMM accumulates
straight into it from TMEM and autograd sees no weight gradient at all.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib


def _use_kernel(t: torch.Tensor) -> bool:
    return _lib.on(t)


def gemm_ref(a, b, *, a_mn=False, b_mn=False, out=None, out_dtype=None, accumulate=False, alpha=1.0):
    """PyTorch reference of ``gemm`` (also the CPU path)."""
    A = a.t() if a_mn else a
    B = b if b_mn else b.t()
    res = (A.float() @ B.float()) * alpha
    out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
    if out is not None:
        if accumulate:
            out.add_(res.to(out.dtype))
        else:
            out.copy_(res.to(out.dtype))
        return out
    return res.to(out_dtype)


def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, accumulate: bool = False,
         alpha: float = 1.0, bn: int = 0, max_ctas: int = 0, bias: torch.Tensor | None = None,
         residual: torch.Tensor | None = None, mt: int = 0) -> torch.Tensor:
    """``out[M, N] (+)= alpha * A @ B^T (+ bias) (+ residual)`` in the operand layouts described in the module
    docstring. ``bias [N]`` (fp32) and ``residual [M, N]`` (dtype of ``out``) are added in the GEMM's epilogue."""
    if not _use_kernel(a):
        if bias is None and residual is None:
            return gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out=out, out_dtype=out_dtype, accumulate=accumulate,
                            alpha=alpha)
        y = gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, out_dtype=torch.float32, alpha=alpha)
        if bias is not None:
            y = y + bias.float()
        if residual is not None:
            y = y + residual.float()
        if out is None:
            return y.to(out_dtype or a.dtype)
        out.copy_((y + out.float()) if accumulate else y)
        return out
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "kernel path is bf16"
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty((M, N), device=a.device, dtype=out_dtype or torch.bfloat16)
    assert out.shape == (M, N) and out.stride(1) == 1
    args = _lib.GemmArgs()
    args.A, args.B, args.C = a.data_ptr(), b.data_ptr(), out.data_ptr()
    args.lda, args.ldb, args.ldc = a.stride(0), b.stride(0), out.stride(0)
    args.a_rows, args.b_rows = a.shape[0], b.shape[0]
    args.M, args.N, args.K = M, N, K
    args.a_mn, args.b_mn = int(a_mn), int(b_mn)
    args.out_f32 = int(out.dtype == torch.float32)
    assert out.dtype in (torch.float32, torch.bfloat16)
    args.accumulate = int(accumulate)
    args.alpha = alpha
    args.bn, args.max_ctas, args.mt = bn, max_ctas, mt   # mt: 0 = choose; 2 = 256-row tiles (dense / K-grouped forms)
    if bias is not None:
        assert bias.dtype == torch.float32 and bias.numel() == N and bias.is_contiguous()
        args.bias = bias.data_ptr()
    if residual is not None:
        assert not accumulate and residual.shape == (M, N) and residual.dtype == out.dtype and residual.stride(1) == 1
        args.accumulate, args.Cin, args.ldcin = 1, residual.data_ptr(), residual.stride(0)
    rc = _lib.lib().np_gemm_bf16(C.byref(args), C.c_void_p(_lib.stream()))
    if rc != 0:
        raise _lib.KernelError(
            f"gemm_bf16 failed with code {rc}: M={M} N={N} K={K} a_mn={a_mn} b_mn={b_mn} a={tuple(a.shape)}/"
            f"{a.stride()} b={tuple(b.shape)}/{b.stride()} out={tuple(out.shape)}/{out.stride()} {out.dtype} "
            f"ptrs={a.data_ptr() % 256},{b.data_ptr() % 256},{out.data_ptr() % 256} bn={bn}")
    _lib.LAUNCHES += 1
    return out


def gemm_swiglu(x: torch.Tensor, w_gate: torch.Tensor, w_up: torch.Tensor, *, save_gu: bool = True):
    """``h = silu(x @ w_gate.T) * (x @ w_up.T)`` in one kernel; optionally also returns ``[gate | up]``.

    The B tile of the GEMM is 128 gate rows + 128 up rows, so both pre-activations sit side by side in
    TMEM and the epilogue applies SwiGLU before anything reaches HBM.
    """
    M, K = x.shape
    F = w_gate.shape[0]
    if not _use_kernel(x):
        g = x.float() @ w_gate.float().t()
        u = x.float() @ w_up.float().t()
        h = (torch.nn.functional.silu(g) * u).to(x.dtype)
        return h, (torch.cat([g, u], dim=1).to(x.dtype) if save_gu else None)
    assert w_gate.stride(0) == w_up.stride(0) and w_gate.shape == w_up.shape
    h = torch.empty((M, F), device=x.device, dtype=torch.bfloat16)
    gu = torch.empty((M, 2 * F), device=x.device, dtype=torch.bfloat16) if save_gu else None
    args = _lib.GemmArgs()
    args.A, args.B, args.B2, args.C = x.data_ptr(), w_gate.data_ptr(), w_up.data_ptr(), h.data_ptr()
    args.C2 = gu.data_ptr() if gu is not None else None
    args.lda, args.ldb, args.ldc, args.ldc2 = x.stride(0), w_gate.stride(0), F, 2 * F
    args.a_rows, args.b_rows = M, F
    args.M, args.N, args.K = M, F, K
    args.epilogue = 1
    args.alpha = 1.0
    _lib.check(_lib.lib().np_gemm_bf16(C.byref(args), C.c_void_p(_lib.stream())), "gemm_swiglu")
    return h, gu


# Zero-bubble pipeline schedules split a backward pass into B (input gradients, on the critical path between
# stages) and W (weight gradients, moved into what would be bubbles). While ``_DEFER`` is a list, every weight-gradient
# GEMM is queued there instead of run; ``run_deferred_wgrads`` executes a queue later. ``SPLIT_MODE`` makes ``linear``
# take its autograd function on every device (CPU included), so that all linear weight gradients are deferrable.
_DEFER: "list | None" = None
SPLIT_MODE = False


class defer_wgrad:
    """Context manager: weight-gradient GEMMs issued inside are appended to ``queue`` as ``(w, dy, x)``."""

    def __init__(self, queue: list):
        self.queue, self._prev = queue, None

    def __enter__(self):
        global _DEFER
        self._prev, _DEFER = _DEFER, self.queue
        return self.queue

    def __exit__(self, *exc):
        global _DEFER
        _DEFER = self._prev
        return False


def run_deferred_wgrads(queue: list) -> None:
    """The W step: run the queued weight-gradient GEMMs (into ``main_grad`` when the weight has one, else into
    ``.grad``) and release the saved activations."""
    with torch.no_grad():      # like the backward pass these GEMMs were taken out of: nothing here is differentiated
        while queue:
            w, dy2, x2 = queue.pop(0)
            g = _wgrad_into(w, dy2, x2)
            if g is not None:
                g = g.to(w.dtype)
                w.grad = g if w.grad is None else w.grad + g


def _wgrad_into(w: torch.Tensor, dy2: torch.Tensor, x2: torch.Tensor):
    """dW[N, K] = dy^T x, accumulated into ``w.main_grad`` when present; returns the autograd grad."""
    if _DEFER is not None and (w.is_leaf or hasattr(w, "main_grad")):
        # a weight that is itself computed (two parameters concatenated for one GEMM) has no ``.grad`` to fill later:
        # its gradient has to go back through autograd now, so only leaves and arena views are deferred
        _DEFER.append((w, dy2, x2))
        return None
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        first = not getattr(w, "_main_grad_dirty", False)
        gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, accumulate=not first)
        w._main_grad_dirty = True
        for q in getattr(w, "_covers", None) or (w,):  # a fused view stands for several parameters
            q._main_grad_dirty = True
            cb = getattr(q, "_grad_ready_cb", None)      # the arena's overlapped gradient reduction (optim/arena.py)
            if cb is not None:
                cb(q)
        return None
    return gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype if w.is_cuda else None)


class _Linear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w):
        ctx.save_for_backward(x, w)
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w)
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(x.shape)
        dw = _wgrad_into(w, dy2, x2) if (ctx.needs_input_grad[1] or hasattr(w, "main_grad")) else None
        return dx, dw


class _LinearBias(torch.autograd.Function):
    """``x @ w.T + bias`` with the bias added in the GEMM's epilogue."""

    @staticmethod
    def forward(ctx, x, w, bias):
        ctx.save_for_backward(x, w)
        ctx.bias_dtype = bias.dtype
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, bias=bias.detach().float().contiguous())
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = gemm(dy2, w, b_mn=True).reshape(x.shape) if ctx.needs_input_grad[0] else None
        dw = _wgrad_into(w, dy2, x2) if (ctx.needs_input_grad[1] or hasattr(w, "main_grad")) else None
        db = dy2.float().sum(0).to(ctx.bias_dtype) if ctx.needs_input_grad[2] else None
        return dx, dw, db


def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None) -> torch.Tensor:
    """``x @ w.T (+ bias)``; tcgen05 kernels for bf16 CUDA tensors, ``F.linear`` otherwise."""
    if SPLIT_MODE and not (_lib.on(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16):
        # same math through the autograd function whose weight gradient can be deferred
        xx = x if x.dtype == w.dtype else x.to(w.dtype)
        return _Linear.apply(xx, w) if bias is None else _LinearBias.apply(xx, w, bias)
    if _lib.on(x) and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16:
        rt = getattr(w, "_fsdp_rt", None)
        if rt is not None:  # row-sharded weight: all-gather inside the GEMM, reduce-scattered weight gradient
            from .fsdp_fused import sharded_linear

            y = sharded_linear(x, w, rt)
            return y if bias is None else y + bias
        rec = getattr(w, "_fp8_recipe", None)
        if rec is not None:  # weight tagged by fp8.training.apply_fp8: forward GEMM on e4m3 operands
            if rec == "mxfp8":
                from .gemm_mxfp8 import mx_linear, mx_linear_supported

                if mx_linear_supported(x, w):
                    return mx_linear(x, w, bias)
            else:
                from .gemm_fp8 import fp8_block_linear, fp8_block_linear_supported

                if fp8_block_linear_supported(x, w):
                    return fp8_block_linear(x, w, bias)
        if bias is not None:
            return _LinearBias.apply(x, w, bias)
        return _Linear.apply(x, w)
    return torch.nn.functional.linear(x, w, bias)
