"""Re-export of ``fp8_flow_moe.recipes`` (reference: fp8/recipes.py:3-7)."""
from fp8_flow_moe.recipes import BlockScalingGranularity, FP8RecipeConfig, FP8RecipeType  # noqa: F401
