"""RMSNorm module (reference: model/norm.py:18-49).

The weight is kept in fp32 whatever the model dtype (it is tiny, and the fused kernel reads fp32
weights); bf16 CUDA activations go through ``ops.norm.rms_norm``.
"""
from __future__ import annotations

import torch
import torch.nn as nn

from ..ops.norm import rms_norm


class RMSNorm(nn.Module):
    def __init__(self, size: int, eps: float = 1e-6, device=None, dtype=None, full_precision: bool = True):
        """``full_precision`` is accepted for the reference's signature (model/norm.py:26): the statistics are always
        accumulated in fp32 here, in the kernel as on the PyTorch path, so the flag changes nothing."""
        super().__init__()
        self.size = size
        self.eps = eps
        self.full_precision = True
        self.weight = nn.Parameter(torch.ones(size, device=device, dtype=torch.float32))

    def _apply(self, fn, recurse=True):  # keep the weight fp32 under .to(bf16) / .bfloat16()
        super()._apply(fn, recurse)
        if self.weight.is_floating_point() and self.weight.dtype != torch.float32:
            self.weight.data = self.weight.data.float()
        return self

    def forward(self, x: torch.Tensor, residual: torch.Tensor | None = None):
        """``norm(x)``; with ``residual`` returns ``(norm(x + residual), x + residual)``."""
        return rms_norm(x, self.weight, self.eps, residual)

    def extra_repr(self) -> str:
        return f"{self.size}, eps={self.eps}"
