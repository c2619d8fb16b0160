"""Checkpointing."""
from .distributed import CheckpointConfig, DistributedCheckpointer

__all__ = ["DistributedCheckpointer", "CheckpointConfig"]
