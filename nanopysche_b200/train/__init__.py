"""Training runtime."""
from .data import DistributedDataLoader, DistributedDataset, create_distributed_loader
from .scheduler import CosineWithWarmup, WarmupStableDecay
from .trainer import Trainer, TrainingConfig

__all__ = ["Trainer", "TrainingConfig", "DistributedDataset", "DistributedDataLoader", "create_distributed_loader",
           "CosineWithWarmup", "WarmupStableDecay"]
