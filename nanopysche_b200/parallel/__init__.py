"""Parallelism engines: device mesh, TP, FSDP/AC, CP (ring / Ulysses), PP (schedules + runtime),
auto-schedule, symmetric memory. Mirrors the reference's ``distributed`` package plus ``parallel.py``."""
from .context_parallel import ContextParallelConfig, RingAttention
from .mesh import (MeshDimName, ParallelDims, build_world_mesh, get_cp_mesh, get_dp_mesh, get_dp_model_mesh,
                   get_ep_mesh, get_pp_mesh, get_tp_mesh, get_world_mesh, reset_world_mesh)
from .pipeline_parallel import (DualPipeSchedule, GPipeSchedule, OneForwardOneBackwardSchedule, PipelineStage,
                                ZeroBubbleSchedule, compute_bubble_fraction, validate_schedule)

__all__ = ["PipelineStage", "GPipeSchedule", "OneForwardOneBackwardSchedule", "DualPipeSchedule",
           "ZeroBubbleSchedule", "compute_bubble_fraction", "validate_schedule", "RingAttention",
           "ContextParallelConfig", "MeshDimName", "ParallelDims", "build_world_mesh", "get_world_mesh",
           "reset_world_mesh", "get_dp_model_mesh", "get_dp_mesh", "get_tp_mesh", "get_cp_mesh", "get_pp_mesh",
           "get_ep_mesh"]
