"""FP8 support: re-exports of the standalone ``fp8_flow_moe`` package plus dense-layer FP8 training
(reference: fp8/__init__.py:8-45)."""
from fp8_flow_moe import (BlockScalingGranularity, FP8FlowMoECompute, FP8FlowMoEConfig, FP8RecipeConfig,
                          FP8RecipeType, dequantize_from_fp8, fp8_grouped_gemm, fused_permute_pad,
                          fused_silu_multiply_quantize, fused_swiglu_quantize, fused_unpermute_unpad,
                          quantize_to_fp8, scaling_aware_transpose)
from fp8_flow_moe.flow_moe import FP8_BLOCK_SIZE

from .training import FP8Config, apply_fp8, precompute_fp8_dynamic_scales

__all__ = ["FP8Config", "apply_fp8", "precompute_fp8_dynamic_scales", "FP8FlowMoEConfig", "FP8FlowMoECompute",
           "FP8RecipeConfig", "FP8RecipeType", "BlockScalingGranularity", "quantize_to_fp8", "dequantize_from_fp8",
           "scaling_aware_transpose", "fused_swiglu_quantize", "fused_silu_multiply_quantize", "fused_permute_pad",
           "fused_unpermute_unpad", "fp8_grouped_gemm", "FP8_BLOCK_SIZE"]
