"""FP8 training for dense Linear layers (reference: fp8/training.py:54-137, which delegates to
torchao's ``convert_to_float8_training``).

Here ``apply_fp8`` swaps eligible ``nn.Linear`` modules for ``Float8Linear`` and tags their weights with the
recipe (``weight._fp8_recipe``): e4m3 forward operands with dynamic scales - ``blockwise`` (1x128 activations,
128x128 weights, fp32 scales) or ``mxfp8`` (1x32 blocks, power-of-two scales) - and gradients in bf16 (the
reference's e5m2 backward dtype is accepted and recorded). On bf16 CUDA tensors ``ops.gemm.linear`` sends a tagged
weight to the fp8 tcgen05 GEMM of its recipe (``csrc/gemm_fp8_sm100.cu``, ``csrc/gemm_mxfp8_sm100.cu``), whether
the layer is called as a module or its weight is used by a fused block; elsewhere the quantise-dequantise pair
is applied around the GEMM, which gives the numerics of fp8 operands with fp32 accumulation on every device.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch
import torch.nn as nn

from fp8_flow_moe import ops as fp8_ops


@dataclass
class FP8Config:
    # fields, order and defaults of the reference (fp8/training.py:70-76). ``recipe_name``: "mxfp8" selects the 1x32
    # e8m0 recipe, every other value (the reference's "max" / "delayed" included) the 1x128 / 128x128 block-scaled
    # one; the dtype names are kept for the record (forward operands are e4m3 here, gradients stay bf16)
    enabled: bool = False
    forward_dtype: str = "float8_e4m3fn"
    backward_dtype: str = "float8_e5m2"
    recipe_name: str = "max"
    force_recompute_fp8_weight_in_bwd: bool = True
    cast_input_text: bool = True            # activations are always cast here
    filter_fn: Optional[str] = None         # substring a module's name must contain
    ignored_modules: List[str] = field(default_factory=lambda: ["lm_head", "gate"])
    min_features: int = 128

    def build_torchao_config(self):
        """The reference hands its linears to torchao (fp8/training.py:78-90). Here the fp8 linears run on this
        package's own block-scaled kernels and nothing is delegated, so there is no torchao object to build: ``None``,
        which is also what the reference returns when torchao is not installed."""
        return None


class _QDQ(torch.autograd.Function):
    """Quantise-dequantise with a straight-through gradient."""

    @staticmethod
    def forward(ctx, x, weight_mode):
        if weight_mode:
            q, s = fp8_ops.quantize_weight_blockwise(x)
        else:
            q, s = fp8_ops.quantize_to_fp8(x.reshape(-1, x.shape[-1]))
            q = q.reshape(x.shape)
            s = s.reshape(*x.shape[:-1], -1)
        return fp8_ops.dequantize_from_fp8(q, s, dtype=x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None


class _QDQmx(torch.autograd.Function):
    """MXFP8 quantise-dequantise (1x32 blocks along the last dimension) with a straight-through gradient."""

    @staticmethod
    def forward(ctx, x):
        from ..ops.gemm_mxfp8 import mx_dequantize, mx_quantize_ref

        q, s = mx_quantize_ref(x.reshape(-1, x.shape[-1]))
        return mx_dequantize(q, s).to(x.dtype).reshape(x.shape)

    @staticmethod
    def backward(ctx, g):
        return g


class Float8Linear(nn.Linear):
    def forward(self, x):
        if x.shape[-1] % 128 or self.weight.shape[0] % 128:
            return super().forward(x)
        from ..ops.gemm import linear

        if x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16:
            return linear(x, self.weight, self.bias)  # dispatches on the weight's recipe tag
        if getattr(self.weight, "_fp8_recipe", None) == "mxfp8":
            return nn.functional.linear(_QDQmx.apply(x), _QDQmx.apply(self.weight), self.bias)
        return linear(_QDQ.apply(x, False), _QDQ.apply(self.weight, True), self.bias)


def apply_fp8(model: nn.Module, config: Optional[FP8Config] = None,
              module_filter: Optional[Callable[[nn.Module, str], bool]] = None) -> nn.Module:
    cfg = config or FP8Config(enabled=True)
    if not cfg.enabled:
        return model
    for name, mod in list(model.named_modules()):
        for cname, child in list(mod.named_children()):
            fqn = f"{name}.{cname}" if name else cname
            if type(child) is not nn.Linear:
                continue
            if any(ig in fqn for ig in cfg.ignored_modules) or min(child.in_features, child.out_features) < \
                    cfg.min_features:
                continue
            if module_filter is not None and not module_filter(child, fqn):
                continue
            if cfg.filter_fn and cfg.filter_fn not in fqn:
                continue
            child.__class__ = Float8Linear
            child.weight._fp8_recipe = "mxfp8" if cfg.recipe_name == "mxfp8" else "blockwise"
    model._fp8_config = cfg
    return model


def precompute_fp8_dynamic_scales(model: nn.Module) -> int:
    """Refresh cached weight quantisation after an optimizer step; returns the number of fp8 layers."""
    return sum(1 for m in model.modules() if isinstance(m, Float8Linear))
