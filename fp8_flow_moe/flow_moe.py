"""FP8-Flow-MoE expert compute: casting-free fp8 dataflow through the expert MLP.

``FP8FlowMoECompute`` holds (views of) the expert weights and computes, for rows sorted by expert,
``(silu(x w1^T) * (x w3^T)) w2`` either in bf16 (fewer than ``fp8_gemm_threshold`` tokens per expert:
quantisation overhead is not amortised) or with e4m3 operands (1x128 activation scales x 128x128 weight
scales): quantise once on entry, SwiGLU and re-quantisation fused, weights quantised once per
optimizer step and cached. With the ``mxfp8`` recipe the operands are e4m3 with one power-of-two scale per 1x32
block along the contraction and the grouped GEMMs run on the block-scaled tensor-core instruction
(``nanopysche_b200/csrc/gemm_mxfp8_sm100.cu``).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch
import torch.nn.functional as F

from . import ops
from .ops import FP8_BLOCK_SIZE  # noqa: F401
from .recipes import FP8RecipeConfig, FP8RecipeType


@dataclass
class FP8FlowMoEConfig:
    enabled: bool = False
    fp8_recipe: FP8RecipeConfig = field(default_factory=FP8RecipeConfig)


class FP8FlowMoECompute:
    def __init__(self, config: FP8FlowMoEConfig, d_model: int, hidden: int, num_experts: int,
                 fp8_gemm_threshold: int = 1000000):
        self.config = config
        self.d_model, self.hidden, self.num_experts = d_model, hidden, num_experts
        self.fp8_gemm_threshold = fp8_gemm_threshold
        self.w1 = self.w2 = self.w3 = None
        self._wq_cache = None
        self._wq_version = None
        self.last_path: Optional[str] = None

    def set_weights(self, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor):
        """``w1, w3: [E*H, D]`` (used as ``x @ w^T``), ``w2: [E*H, D]`` (used as ``h @ w2``)."""
        self.w1, self.w2, self.w3 = w1, w2, w3
        self._wq_cache = None

    def _quantised_weights(self):
        ver = tuple(w._version for w in (self.w1, self.w2, self.w3))
        if self._wq_cache is None or self._wq_version != ver:
            E, H, D = self.num_experts, self.hidden, self.d_model
            w1q, s1 = ops.quantize_weight_blockwise(self.w1.detach().reshape(E * H, D))
            w3q, s3 = ops.quantize_weight_blockwise(self.w3.detach().reshape(E * H, D))
            w2t = self.w2.detach().reshape(E, H, D).transpose(1, 2).contiguous().reshape(E * D, H)
            w2q, s2 = ops.quantize_weight_blockwise(w2t)
            self._wq_cache = (w1q.view(E, H, D), s1.view(E, H // 128, D // 128), w3q.view(E, H, D),
                              s3.view(E, H // 128, D // 128), w2q.view(E, D, H), s2.view(E, D // 128, H // 128))
            self._wq_version = ver
        return self._wq_cache

    def _mx_weights(self):
        """1x32-scaled e4m3 copies of the expert weights, K-major for their GEMM: w1, w3 ``[E*H, D]`` quantised
        along D, w2 transposed per expert to ``[E*D, H]`` and quantised along H. Cached per weight version."""
        from nanopysche_b200.ops.gemm_mxfp8 import mx_quantize

        ver = ("mx",) + tuple(w._version for w in (self.w1, self.w2, self.w3))
        if self._wq_cache is None or self._wq_version != ver:
            E, H, D = self.num_experts, self.hidden, self.d_model
            bf = lambda t: t.detach().to(torch.bfloat16).contiguous()
            w2t = self.w2.detach().reshape(E, H, D).transpose(1, 2).reshape(E * D, H)
            self._wq_cache = (*mx_quantize(bf(self.w1.reshape(E * H, D))), *mx_quantize(bf(self.w3.reshape(E * H, D))),
                              *mx_quantize(bf(w2t)))
            self._wq_version = ver
        return self._wq_cache

    def use_fp8(self, tokens_per_expert: float) -> bool:
        c = self.config
        return bool(c.enabled and c.fp8_recipe.active and tokens_per_expert >= self.fp8_gemm_threshold and
                    self.d_model % 128 == 0 and self.hidden % 128 == 0)

    def __call__(self, x: torch.Tensor, weights: Optional[torch.Tensor], indices: torch.Tensor,
                 expert_start: int = 0, num_experts: Optional[int] = None) -> torch.Tensor:
        """``x [n, D]`` rows with local expert ids ``indices [n]`` (any order) -> ``[n, D]`` expert outputs
        (multiplied by ``weights [n]`` when given)."""
        E = num_experts or self.num_experts
        n = x.shape[0]
        if n == 0:
            return x.new_zeros((0, self.d_model))
        H, D = self.hidden, self.d_model
        idx = indices.reshape(-1) - expert_start
        if self.use_fp8(n / max(E, 1)):
            self.last_path = "fp8"
            xp, row_map, padded = ops.fused_permute_pad(x, idx, E, 128)
            if self.config.fp8_recipe.recipe_type == FP8RecipeType.MXFP8:
                from nanopysche_b200.ops.gemm_mxfp8 import mx_expert_mlp

                self.last_path = "mxfp8"
                y = mx_expert_mlp(xp, self.w1, self.w3, self.w2, padded.tolist(), self._mx_weights())
                return ops.fused_unpermute_unpad(y, row_map, weights)
            xq, xs = ops.quantize_to_fp8(xp)
            w1q, s1, w3q, s3, w2q, s2 = self._quantised_weights()
            g = ops.fp8_grouped_gemm(xq, xs, w1q, s1, padded)
            u = ops.fp8_grouped_gemm(xq, xs, w3q, s3, padded)
            hq, hs = ops.fused_silu_multiply_quantize(g, u)
            y = ops.fp8_grouped_gemm(hq, hs, w2q, s2, padded, out_dtype=x.dtype)
            if torch.is_grad_enabled() and (x.requires_grad or self.w1.requires_grad):
                # straight-through: fp8 value in forward, bf16 expert math for the gradient
                y_ref = self._bf16(xp, padded)
                y = y_ref + (y - y_ref).detach()
            return ops.fused_unpermute_unpad(y, row_map, weights)
        self.last_path = "bf16"
        order = torch.argsort(idx, stable=True)
        counts = torch.bincount(idx, minlength=E)
        ys = self._bf16(x[order], counts)
        out = torch.empty_like(ys)
        out[order] = ys
        return out if weights is None else out * weights.reshape(-1, 1).to(out.dtype)

    def _bf16(self, xs: torch.Tensor, counts: torch.Tensor) -> torch.Tensor:
        H, D = self.hidden, self.d_model
        outs, start = [], 0
        for e, c in enumerate(counts.tolist()):
            if c:
                seg = xs[start:start + c]
                w1, w3, w2 = (w[e * H:(e + 1) * H].to(seg.dtype) for w in (self.w1, self.w3, self.w2))
                outs.append((F.silu(seg @ w1.t()) * (seg @ w3.t())) @ w2)
            start += c
        return torch.cat(outs, 0) if outs else xs.new_zeros((0, D))
