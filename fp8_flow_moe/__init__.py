"""fp8_flow_moe: standalone FP8-Flow-MoE operators (no dependency on the training framework).

Blockwise e4m3 quantisation (1x128 activations, 128x128 weights, optional 1x32 power-of-two scales),
scaling-aware transpose, fused SwiGLU+quantise, permute+pad / unpermute+unpad and the block-scaled
grouped GEMM, plus ``FP8FlowMoECompute`` which strings them into the expert MLP with a runtime
bf16 / fp8 switch on tokens per expert.
"""
from .flow_moe import FP8_BLOCK_SIZE, FP8FlowMoECompute, FP8FlowMoEConfig
from .ops import (dequantize_from_fp8, fp8_grouped_gemm, fused_permute_pad, fused_silu_multiply_quantize,
                  fused_swiglu_quantize, fused_unpermute_unpad, quantize_to_fp8, quantize_weight_blockwise,
                  scaling_aware_transpose)
from .recipes import BlockScalingGranularity, FP8RecipeConfig, FP8RecipeType

__version__ = "0.1.0"
__all__ = ["FP8FlowMoEConfig", "FP8FlowMoECompute", "FP8RecipeConfig", "FP8RecipeType", "BlockScalingGranularity",
           "FP8_BLOCK_SIZE", "quantize_to_fp8", "dequantize_from_fp8", "quantize_weight_blockwise",
           "scaling_aware_transpose", "fused_swiglu_quantize", "fused_silu_multiply_quantize", "fused_permute_pad",
           "fused_unpermute_unpad", "fp8_grouped_gemm"]
