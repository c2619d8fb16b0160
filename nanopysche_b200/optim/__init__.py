"""Optimizers: AdamW, the flat-arena fused AdamW, and the DiLoCo gradient compressor."""
from .adamw import AdamW, create_adamw
from .arena import ArenaAdamW, ParamArena
from .diko import DiLoCoCompressor

__all__ = ["AdamW", "create_adamw", "DiLoCoCompressor", "ParamArena", "ArenaAdamW"]
