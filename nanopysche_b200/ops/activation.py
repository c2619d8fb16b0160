"""Gated-linear-unit activations (SwiGLU / GeGLU) on a fused ``[gate | up]`` buffer.

Kernel: csrc/elementwise.cu ``glu_fwd/bwd``; reference math: model/feed_forward.py:64-75
(``w2(act(w1 x) * w3 x)``, act in {silu, gelu_tanh}).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _lib

ACT_IDS = {"silu": 0, "gelu_tanh": 1}


def glu_ref(gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    g, u = gu.float().chunk(2, dim=-1)
    a = F.silu(g) if act == "silu" else F.gelu(g, approximate="tanh")
    return (a * u).to(gu.dtype)


class _GLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, act_id):
        Fh = gu.shape[-1] // 2
        gu2 = gu.reshape(-1, 2 * Fh)
        gu2 = gu2 if gu2.is_contiguous() else gu2.contiguous()
        h = torch.empty((gu2.shape[0], Fh), device=gu.device, dtype=gu.dtype)
        _lib.call("glu_fwd", gu2, h, _lib.LL(gu2.shape[0]), Fh, act_id)
        ctx.save_for_backward(gu2)
        ctx.act_id = act_id
        ctx.shape = gu.shape
        return h.view(*gu.shape[:-1], Fh)

    @staticmethod
    def backward(ctx, dh):
        (gu2,) = ctx.saved_tensors
        Fh = gu2.shape[1] // 2
        dh2 = dh.reshape(-1, Fh)
        dh2 = dh2 if dh2.is_contiguous() else dh2.contiguous()
        dgu = torch.empty_like(gu2)
        _lib.call("glu_bwd", gu2, dh2, dgu, _lib.LL(gu2.shape[0]), Fh, ctx.act_id)
        return dgu.view(ctx.shape), None


def glu_bwd(gu: torch.Tensor, dh: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """Gradient of ``glu`` w.r.t. the ``[gate | up]`` buffer (used by the fused GEMM+SwiGLU path)."""
    if _lib.on(gu) and gu.dtype == torch.bfloat16:
        Fh = gu.shape[-1] // 2
        gu2, dh2 = gu.reshape(-1, 2 * Fh), dh.reshape(-1, Fh).contiguous()
        dgu = torch.empty_like(gu2)
        _lib.call("glu_bwd", gu2, dh2, dgu, _lib.LL(gu2.shape[0]), Fh, ACT_IDS[act])
        return dgu.view(gu.shape)
    g, u = gu.float().chunk(2, dim=-1)
    g = g.detach().requires_grad_(True)
    with torch.enable_grad():
        a = F.silu(g) if act == "silu" else F.gelu(g, approximate="tanh")
    (da,) = torch.autograd.grad(a, g, dh.float() * u)
    return torch.cat([da, dh.float() * a.detach()], dim=-1).to(gu.dtype)


def glu(gu: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """``act(gate) * up`` for ``gu = [gate | up]`` along the last dim."""
    if _lib.on(gu) and gu.dtype == torch.bfloat16 and (gu.shape[-1] // 2) % 8 == 0:
        return _GLU.apply(gu, ACT_IDS[act])
    return glu_ref(gu, act)
