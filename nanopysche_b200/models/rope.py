"""Rotary embeddings (reference: model/rope.py:21-170).

``RotaryEmbedding`` keeps the reference's interface (``forward(seq_len, offset=, device=, dtype=)``
returning full-width ``[S, rot]`` cos/sin) and additionally exposes half-width fp32 tables for the
fused kernel. ``RoPEScalingConfig.rope_type`` selects the reference's piecewise rule (default) or a
true YaRN (NTK-by-parts ramp plus attention scale).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..ops import rope as rope_ops


@dataclass
class RoPEScalingConfig:
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192
    rope_type: str = "piecewise"  # "piecewise" (reference rule) or "yarn"
    beta_fast: float = 32.0
    beta_slow: float = 1.0


class RotaryEmbedding(nn.Module):
    def __init__(self, dim: int, *, base: float = 10000.0, max_seq_len: int = 8192, head_first: bool = True,
                 partial_rotary_factor: float = 1.0, scaling: Optional[RoPEScalingConfig] = None):
        super().__init__()
        self.dim = dim
        self.base = base
        self.max_seq_len = max_seq_len
        self.head_first = head_first
        self.partial_rotary_factor = partial_rotary_factor
        self.scaling = scaling
        self.rotary_dim = int(dim * partial_rotary_factor)
        assert self.rotary_dim % 2 == 0, "rotary dimension must be even"
        inv_freq = 1.0 / (base ** (torch.arange(0, self.rotary_dim, 2).float() / self.rotary_dim))
        self.register_buffer("inv_freq", inv_freq, persistent=False)
        self._half: dict = {}

    def _table_args(self):
        s = self.scaling
        if s is None or s.factor <= 1.0:
            return dict(scaling=None)
        if s.rope_type == "yarn":
            return dict(scaling="yarn", factor=s.factor, orig_len=float(s.original_max_position_embeddings),
                        low_f=s.beta_slow, high_f=s.beta_fast)
        return dict(scaling="piecewise", factor=s.factor, orig_len=float(s.original_max_position_embeddings),
                    low_f=s.low_freq_factor, high_f=s.high_freq_factor)

    def half_tables(self, seq_len: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """fp32 ``[>=seq_len, rot/2]`` cos/sin, cached per device and grown on demand."""
        key = str(device)
        cur = self._half.get(key)
        if cur is None or cur[0].shape[0] < seq_len:
            n = max(seq_len, self.max_seq_len if cur is None else 2 * cur[0].shape[0])
            cur = rope_ops.rope_tables(n, self.rotary_dim, self.base, device=device, **self._table_args())
            self._half[key] = cur
        return cur

    def get_buffers(self, seq_len: int, device, dtype) -> Tuple[torch.Tensor, torch.Tensor]:
        c, s = self.half_tables(seq_len, device)
        return torch.cat([c, c], -1)[:seq_len].to(dtype), torch.cat([s, s], -1)[:seq_len].to(dtype)

    def warmup_cache(self, seq_len: int, device, dtype: torch.dtype = torch.float32):
        self.half_tables(seq_len, device)

    def forward(self, seq_len: int, *, offset: int = 0, device, dtype: torch.dtype = torch.float32):
        cos, sin = self.get_buffers(offset + seq_len, device, dtype)
        return cos[offset:offset + seq_len], sin[offset:offset + seq_len]


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    x1, x2 = x.chunk(2, dim=-1)
    return torch.cat([-x2, x1], dim=-1)


def apply_rotary_emb(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, head_first: bool = True) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin``; x is (B,S,H,D) when ``head_first`` else (B,H,S,D); cos/sin (S, rot)."""
    rot = cos.shape[-1]
    if head_first:
        c, s = cos[None, :, None, :], sin[None, :, None, :]
    else:
        c, s = cos[None, None, :, :], sin[None, None, :, :]
    xr, xp = x[..., :rot], x[..., rot:]
    out = xr * c.to(x.dtype) + rotate_half(xr) * s.to(x.dtype)
    return torch.cat([out, xp], dim=-1) if xp.shape[-1] else out
