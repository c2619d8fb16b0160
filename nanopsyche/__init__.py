"""Import-path compatibility with the reference package name.

``import nanopsyche`` and every reference sub-module path (``nanopsyche.model.moe``,
``nanopsyche.distributed.pipeline_runtime``, ``nanopsyche.parallel``, ``nanopsyche.train.trainer`` ...)
resolve to the corresponding ``nanopysche_b200`` module, so code written against the reference
(reference: __init__.py:23-53 and the package layout) runs unchanged on this framework.
"""
import importlib
import sys

import nanopysche_b200 as _impl
from nanopysche_b200 import *  # noqa: F401,F403
from nanopysche_b200 import __all__, __version__  # noqa: F401

_ALIASES = {
    "model": "models", "model.norm": "models.norm", "model.rope": "models.rope",
    "model.attention": "models.attention", "model.feed_forward": "models.feed_forward", "model.moe": "models.moe",
    "model.transformer": "models.transformer", "model.tp_utils": "models.tp_utils",
    "model.protocol": "models.protocol", "model.parallel_adapter": "models.parallel_adapter",
    "distributed": "parallel", "distributed.tensor_parallel": "parallel.tensor_parallel",
    "distributed.fsdp": "parallel.fsdp", "distributed.context_parallel": "parallel.context_parallel",
    "distributed.pipeline_parallel": "parallel.pipeline_parallel",
    "distributed.pipeline_runtime": "parallel.pipeline_runtime", "distributed.auto_schedule": "parallel.auto_schedule",
    "parallel": "parallel.mesh", "parallelize": "parallelize", "config": "config", "cli": "cli",
    "model_factory": "model_factory", "bench_utils": "bench_utils", "train": "train", "train.trainer": "train.trainer",
    "train.data": "train.data", "train.scheduler": "train.scheduler", "train.callbacks": "train.callbacks",
    "train.callbacks.base": "train.callbacks.base", "train.callbacks.speed_monitor": "train.callbacks.speed_monitor",
    "train.callbacks.gpu_memory_monitor": "train.callbacks.gpu_memory_monitor",
    "train.callbacks.stability_monitor": "train.callbacks.stability_monitor",
    "train.callbacks.console_logger": "train.callbacks.console_logger",
    "train.callbacks.wandb_logger": "train.callbacks.wandb_logger", "train.callbacks.profiler": "train.callbacks.profiler",
    "optim": "optim", "optim.adamw": "optim.adamw", "optim.diko": "optim.diko", "checkpoint": "checkpoint",
    "checkpoint.distributed": "checkpoint.distributed", "fault_tolerance": "fault_tolerance",
    "fault_tolerance.checkpoint": "fault_tolerance.checkpoint",
    "fault_tolerance.hang_detection": "fault_tolerance.hang_detection", "fp8": "fp8", "fp8.training": "fp8.training",
    "fp8.flow_moe": "fp8.flow_moe", "fp8.recipes": "fp8.recipes",
}

for _ref, _ours in _ALIASES.items():
    _mod = importlib.import_module("nanopysche_b200." + _ours)
    sys.modules["nanopsyche." + _ref] = _mod
    if "." not in _ref:
        globals()[_ref] = _mod
