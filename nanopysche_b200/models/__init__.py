"""Model layer: norms, RoPE, attention, feed-forward, MoE, blocks and the Transformer."""
from .attention import Attention
from .feed_forward import ActivationFunction, FeedForward
from .moe import MoEBase, MoERouter
from .norm import RMSNorm
from .rope import RoPEScalingConfig, RotaryEmbedding, apply_rotary_emb
from .transformer import MoEHybridTransformerBlock, Transformer, TransformerBlock

__all__ = ["RMSNorm", "RotaryEmbedding", "RoPEScalingConfig", "apply_rotary_emb", "Attention", "FeedForward",
           "ActivationFunction", "MoEBase", "MoERouter", "TransformerBlock", "MoEHybridTransformerBlock",
           "Transformer"]
