"""FP8 recipes of FP8-Flow-MoE: which tensors are quantised and at what granularity."""
from __future__ import annotations

from dataclasses import dataclass
from enum import Enum


class FP8RecipeType(str, Enum):
    NONE = "none"
    BLOCKWISE = "blockwise"   # e4m3, 1x128 activation blocks x 128x128 weight blocks, fp32 scales
    MXFP8 = "mxfp8"           # e4m3, 1x32 blocks, power-of-two (UE8M0) scales
    FLOW_MOE = "flow_moe"     # blockwise + quantised dispatch (fp8 on the wire) + fused permute/pad


class BlockScalingGranularity(str, Enum):
    TENSOR = "tensor"
    ROW = "row"
    BLOCK_1x128 = "1x128"
    BLOCK_128x128 = "128x128"
    BLOCK_1x32 = "1x32"


@dataclass
class FP8RecipeConfig:
    enabled: bool = False
    recipe_type: FP8RecipeType = FP8RecipeType.NONE
    activation_granularity: BlockScalingGranularity = BlockScalingGranularity.BLOCK_1x128
    weight_granularity: BlockScalingGranularity = BlockScalingGranularity.BLOCK_128x128

    def __post_init__(self):
        self.recipe_type = FP8RecipeType(self.recipe_type)
        if self.recipe_type == FP8RecipeType.MXFP8:
            self.activation_granularity = BlockScalingGranularity.BLOCK_1x32
            self.weight_granularity = BlockScalingGranularity.BLOCK_1x32

    @property
    def block_size(self) -> int:
        return 32 if self.recipe_type == FP8RecipeType.MXFP8 else 128

    @property
    def active(self) -> bool:
        return self.enabled and self.recipe_type != FP8RecipeType.NONE
