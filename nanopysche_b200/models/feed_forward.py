"""Gated feed-forward network, SwiGLU or GeGLU (reference: model/feed_forward.py:29-116).

``w2(act(w1 x) * w3 x)`` with the reference's parameter names. On bf16 CUDA tensors the gate and up
projections run as one tcgen05 GEMM over the fused ``[w1; w3]`` weight view (set up by the parameter
arena) followed by the GLU kernel; TP shards w1/w3 column-wise and w2 row-wise with both Megatron
conjugate operators.
"""
from __future__ import annotations

from enum import Enum
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import _lib
from ..ops import activation as act_ops
from ..ops import gemm as gemm_ops
from .tp_utils import copy_to_tp_region, differentiable_all_reduce


class ActivationFunction(str, Enum):
    silu = "silu"
    gelu_tanh = "gelu_tanh"


class FeedForward(nn.Module):
    def __init__(self, *, d_model: int, hidden_size: Optional[int] = None, bias: bool = False,
                 activation: ActivationFunction = ActivationFunction.silu, dtype=None, device=None):
        super().__init__()
        hidden = hidden_size or int(8 / 3 * d_model)
        hidden = ((hidden + 255) // 256) * 256 if hidden_size is None else hidden
        self.d_model, self.hidden_size = d_model, hidden
        self.activation = ActivationFunction(activation)
        kw = dict(dtype=dtype, device=device)
        # registered in the reference's order (model/feed_forward.py: w1, w2, w3), which is the order optimizer state is
        # stored in; the flat parameter arena lays w1 and w3 out back to back by itself (one gate|up GEMM)
        self.w1 = nn.Linear(d_model, hidden, bias=bias, **kw)
        self.w2 = nn.Linear(hidden, d_model, bias=bias, **kw)
        self.w3 = nn.Linear(d_model, hidden, bias=bias, **kw)
        self._tp_size = 1
        self._tp_group = None
        self._fused_w13: Optional[torch.Tensor] = None
        self._tp_rt = None  # ops.tp_fused.TPRuntime when the fused sequence-parallel TP path is on

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        act = self.activation.value
        from ..ops import tp_fused

        if tp_fused.active(self._tp_rt, x) and self.w1.bias is None:

            rt = self._tp_rt
            w13 = self._fused_w13 if self._fused_w13 is not None else torch.cat([self.w1.weight, self.w3.weight], 0)
            h = act_ops.glu(tp_fused.ag_linear(x.reshape(-1, x.shape[-1]), w13, rt), act)
            return tp_fused.linear_rs(h, self.w2.weight, rt).view(*x.shape[:-1], -1)
        x = copy_to_tp_region(x, self._tp_group, self._tp_size)
        fused = self._fused_w13
        if fused is not None and _lib.on(x) and x.dtype == fused.dtype and self.w1.bias is None:
            h = act_ops.glu(gemm_ops.linear(x, fused), act)
        elif _lib.on(x) and x.dtype == torch.bfloat16 and self.w1.bias is None:
            gu = torch.cat([gemm_ops.linear(x, self.w1.weight), gemm_ops.linear(x, self.w3.weight)], dim=-1)
            h = act_ops.glu(gu, act)
        else:
            g = gemm_ops.linear(x, self.w1.weight, self.w1.bias)
            a = F.silu(g) if act == "silu" else F.gelu(g, approximate="tanh")
            h = a * gemm_ops.linear(x, self.w3.weight, self.w3.bias)
        out = gemm_ops.linear(h, self.w2.weight, None)
        out = differentiable_all_reduce(out, self._tp_group, self._tp_size)
        if self.w2.bias is not None:
            out = out + self.w2.bias
        return out

    def apply_tp(self, tp_mesh, **_):
        import torch.distributed as dist

        group = tp_mesh.get_group() if hasattr(tp_mesh, "get_group") else tp_mesh
        tp, rank = dist.get_world_size(group), dist.get_rank(group)
        if tp <= 1:
            return
        assert self.hidden_size % tp == 0
        self._tp_size, self._tp_group = tp, group
        n = self.hidden_size // tp
        for lin in (self.w1, self.w3):
            lin.weight = nn.Parameter(lin.weight.data[rank * n:(rank + 1) * n].clone())
            if lin.bias is not None:
                lin.bias = nn.Parameter(lin.bias.data[rank * n:(rank + 1) * n].clone())
            lin.out_features = n
        self.w2.weight = nn.Parameter(self.w2.weight.data[:, rank * n:(rank + 1) * n].clone())
        self.w2.in_features = n
        for lin in (self.w1, self.w3, self.w2):
            lin.weight._tp_sharded = group
            if lin.bias is not None and lin is not self.w2:
                lin.bias._tp_sharded = group
        self._fused_w13 = None
