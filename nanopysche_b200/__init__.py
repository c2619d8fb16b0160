"""nanopysche_b200: a Blackwell-native (sm_100a) 5-D-parallel LLM training framework with the
capabilities and public API of nanopsyche (reference: __init__.py:23-53).

Layout: ``models/`` (modules), ``ops/`` (autograd ops over the in-tree CUDA kernels, each with a
PyTorch reference), ``parallel/`` (mesh, TP, CP, PP, FSDP, symmetric memory), ``train/``, ``optim/``,
``checkpoint/``, ``fault_tolerance/``, ``fp8/``, ``csrc/`` (CUDA sources), ``lib/`` (built library).
"""
from .config import ExperimentConfig, TrainingConfig, TransformerConfig
from .model_factory import ModelBuildContext, build_model, load_factory
from .models import Attention, FeedForward, MoEBase, RMSNorm, Transformer, TransformerBlock
from .models.parallel_adapter import ensure_parallel_hooks
from .train import Trainer

__version__ = "0.1.0"
__all__ = ["Transformer", "TransformerBlock", "RMSNorm", "Attention", "FeedForward", "MoEBase", "Trainer",
           "ExperimentConfig", "TransformerConfig", "TrainingConfig", "ModelBuildContext", "build_model",
           "load_factory", "ensure_parallel_hooks"]
