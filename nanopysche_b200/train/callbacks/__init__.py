"""Training callbacks."""
from .base import Callback
from .console_logger import ConsoleLoggerCallback
from .gpu_memory_monitor import GPUMemoryMonitorCallback
from .profiler import ProfilerCallback
from .speed_monitor import SpeedMonitorCallback
from .stability_monitor import StabilityMonitorCallback
from .throughput_summary import ThroughputSummaryCallback
from .validation import ValidationCallback
from .wandb_logger import WandBCallback

__all__ = ["Callback", "SpeedMonitorCallback", "GPUMemoryMonitorCallback", "WandBCallback", "ConsoleLoggerCallback",
           "ProfilerCallback", "StabilityMonitorCallback", "ValidationCallback", "ThroughputSummaryCallback"]
