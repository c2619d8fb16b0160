"""Fault tolerance: resumable checkpoints and hang detection."""
from .checkpoint import FaultTolerantCheckpointer
from .hang_detection import CommTimeoutError, HangDetector, HeartbeatCoordinator, PeerLeftError

__all__ = ["FaultTolerantCheckpointer", "HangDetector", "HeartbeatCoordinator", "CommTimeoutError", "PeerLeftError"]
