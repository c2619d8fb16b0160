"""``parallelize_model``: composes every parallelism dimension in a fixed order
(reference: parallelize.py:56-194).

Order: ensure hooks -> warn unsupported -> PP -> FP8 -> CP -> TP (+ fused "async" TP) -> EP
(+ FP8-Flow-MoE recipe on every MoE layer) -> activation checkpointing -> compile (no-op marker) ->
FSDP / sharded data parallelism -> weight init for models that ask for it. FSDP stays last so the
parameters it shards are the final (TP / EP-sliced) ones; optimizers must be built *after* this call.
"""
from __future__ import annotations

import logging
from typing import Optional

import torch
import torch.nn as nn

from .models.moe import MoEBase
from .models.parallel_adapter import ensure_parallel_hooks
from .models.protocol import warn_unsupported_parallelism
from .parallel.context_parallel import ContextParallelConfig
from .parallel.fsdp import DataParallelConfig, apply_activation_checkpointing, apply_generic_fsdp
from .parallel.mesh import (MeshDimName, get_cp_mesh, get_dp_model_mesh, get_ep_mesh, get_hsdp_groups, get_pp_mesh,
                            get_replica_group, get_tp_mesh)
from .parallel.tensor_parallel import TensorParallelConfig

log = logging.getLogger(__name__)


_PP_SCHEDULE_NAMES = {"1f1b": "1F1B", "gpipe": "GPipe", "dualpipe": "DualPipe", "interleaved": "Interleaved1F1B",
                      "interleaved1f1b": "Interleaved1F1B", "loopedbfs": "LoopedBFS", "zb": "InterleavedZeroBubble",
                      "zero_bubble": "InterleavedZeroBubble", "zerobubble": "InterleavedZeroBubble",
                      "interleavedzerobubble": "InterleavedZeroBubble", "zbv": "ZBVZeroBubble",
                      "zbvzerobubble": "ZBVZeroBubble"}


def runtime_pp_config(pp_config):
    """Either of the two ``PipelineParallelConfig`` classes (the reference has both: distributed/pipeline_parallel.py
    with a schedule *name*, distributed/pipeline_runtime.py with a schedule *type*) as the runtime one."""
    from .parallel.pipeline_runtime import PipelineParallelConfig as RuntimeConfig
    from .parallel.pipeline_runtime import PipelineScheduleType

    if isinstance(pp_config, RuntimeConfig):
        return pp_config
    name = str(getattr(pp_config.schedule, "value", pp_config.schedule))
    st = PipelineScheduleType(_PP_SCHEDULE_NAMES.get(name.lower(), name))
    return RuntimeConfig(degree=pp_config.degree, schedule=st, num_microbatches=pp_config.num_microbatches)


def parallelize_model(model: nn.Module, *, world_mesh, device: Optional[torch.device] = None,
                      max_sequence_length: Optional[int] = None, tp_config: Optional[TensorParallelConfig] = None,
                      cp_config: Optional[ContextParallelConfig] = None, pp_config=None,
                      dp_config: Optional[DataParallelConfig] = None, fp8_config=None, moe_fp8_recipe: str = "none",
                      moe_fp8_gemm_threshold: int = 1000000, compile_model: bool = False,
                      ac_mode: Optional[str] = None, ac_block_interval: Optional[int] = None) -> nn.Module:
    model = ensure_parallel_hooks(model)
    names = tuple(world_mesh.mesh_dim_names or ()) if world_mesh is not None else ()
    ep_requested = MeshDimName.ep in names
    warn_unsupported_parallelism(model, tp=2 if tp_config else 1, cp=2 if cp_config else 1, pp=2 if pp_config else 1,
                                 ep=2 if ep_requested else 1, fsdp=dp_config is not None, compile=compile_model)
    if pp_config is not None and getattr(pp_config, "degree", 1) > 1:
        log.info("  Applying PP (degree=%d)", pp_config.degree)
        rt_cfg = runtime_pp_config(pp_config)
        pp_mesh = get_pp_mesh(world_mesh)
        if rt_cfg.stages_per_rank() == 1 or not hasattr(model, "n_layers"):
            model.apply_pp(pp_mesh)
            model._pp_config = rt_cfg
        else:
            # interleaved / zero-bubble V / DualPipe: this rank runs two stages; the model becomes a container of them
            from .parallel.pipeline_runtime import PipelineStages, split_model

            group = pp_mesh.get_group() if hasattr(pp_mesh, "get_group") else pp_mesh
            model = PipelineStages(split_model(model, pp_mesh, rt_cfg, device=device), group, rt_cfg)
    if fp8_config is not None and fp8_config.enabled:
        from .fp8.training import apply_fp8

        log.info("  Applying FP8")
        model = apply_fp8(model, config=fp8_config)
    if cp_config is not None and cp_config.degree > 1:
        log.info("  Applying CP (degree=%d)", cp_config.degree)
        model.apply_cp(get_cp_mesh(world_mesh), ring=cp_config.ring and not cp_config.ulysses,
                       uly=cp_config.ulysses)
    if tp_config is not None and tp_config.degree > 1:
        log.info("  Applying TP (degree=%d)", tp_config.degree)
        tp_mesh = get_tp_mesh(world_mesh)
        # "async TP": the sequence-parallel layout with the all-gather inside the column-parallel GEMMs and the
        # reduce-scatter behind the row-parallel ones (ops/tp_fused.py); needs CUDA peer memory and a model whose
        # apply_tp knows the switch, otherwise the plain all-reduce form
        fused = tp_config.maybe_enable_async_tp(tp_mesh) and device is not None and \
            torch.device(device).type == "cuda"
        # without the fused kernels (CPU, or not asked for) ``sequence_parallel`` gives the same row-shard layout
        # through all-gather / reduce-scatter collectives; async TP that cannot be fused falls back to it as well
        seq_par = bool(getattr(tp_config, "sequence_parallel", False) or (tp_config.enable_async and not fused))
        try:
            if fused:
                model.apply_tp(tp_mesh, fused=True)
            elif seq_par:
                model.apply_tp(tp_mesh, sequence_parallel=True)
            else:
                model.apply_tp(tp_mesh)
        except TypeError:
            model.apply_tp(tp_mesh)
            fused = seq_par = False
        if tp_config.enable_async and not fused:
            log.warning("  async TP requested but the fused kernels are not available here: %s",
                        "sequence parallelism through library collectives" if seq_par else "plain all-reduces")
        model._tp_async = bool(fused)
        model._tp_sequence_parallel = bool(fused or seq_par)
    if ep_requested:
        log.info("  Applying EP")
        model.apply_ep(get_ep_mesh(world_mesh))
    if moe_fp8_recipe != "none":
        for module in model.modules():
            if isinstance(module, MoEBase):
                module.apply_fp8_flow_moe(True, moe_fp8_recipe, moe_fp8_gemm_threshold)
    if ac_mode is not None:
        apply_activation_checkpointing(model, mode=ac_mode, block_interval=ac_block_interval)
    if compile_model:
        model.apply_compile()
    if dp_config is not None:
        dp_mesh = get_dp_model_mesh(world_mesh)
        backend = getattr(dp_config, "backend", "auto")
        use_arena = backend == "arena" or (backend == "auto" and device is not None and
                                           torch.device(device).type == "cuda")
        if backend == "sharded" and tp_config is not None and tp_config.degree > 1:
            # the fused tensor-parallel linears read their weights directly (ops/tp_fused.py)
            log.warning("  row-sharded linears are not combined with tensor parallelism: using the arena's ZeRO step")
            backend = "arena"
        if backend == "sharded" and device is not None and torch.device(device).type == "cuda":
            from .parallel.fsdp import fully_shard_linears

            grp = dp_mesh.get_group() if hasattr(dp_mesh, "get_group") else dp_mesh
            if grp is not None:
                fully_shard_linears(model, grp, device=device)
            use_arena = True
        if use_arena:
            # sharded optimizer state + fused reduce-scatter/AdamW/all-gather: set up by engine.prepare_training
            model._dp_mesh_for_arena = dp_mesh
            shard_g, rep_g = get_hsdp_groups(world_mesh)
            if rep_g is not None:      # HSDP: shard over dp_shard, replicate over dp_replicate
                model._replica_group, model._replicate_group = shard_g, rep_g
            else:
                model._replica_group = get_replica_group(world_mesh)   # read by engine.prepare_training
            model._needs_grad_sync = True
        else:
            # FSDP2 shards (and averages gradients) over the dp dims only. Expert-parallel peers read other batches
            # and context-parallel peers other parts of each sequence, so the gradients still have to be combined over
            # those dims: Trainer._sync_fsdp_extra_dims does it after the backward pass. Under sequence-parallel TP
            # the same pass sums the partial gradients (norms, embeddings, routers, MoE weights) over the TP group: FSDP2
            # replaces the parameter objects, so the hooks that do it otherwise never fire.
            names_ = tuple(world_mesh.mesh_dim_names or ()) if world_mesh is not None else ()
            extra = {}
            if getattr(model, "_tp_sequence_parallel", False):
                extra["sp"] = get_tp_mesh(world_mesh).get_group()
            if MeshDimName.ep in names_ and world_mesh[MeshDimName.ep].size() > 1:
                extra["ep"] = world_mesh[MeshDimName.ep].get_group()
            if MeshDimName.cp in names_ and world_mesh[MeshDimName.cp].size() > 1:
                extra["cp"] = world_mesh[MeshDimName.cp].get_group()
            if hasattr(model, "apply_fsdp"):
                model.apply_fsdp(dp_mesh=dp_mesh, param_dtype=dp_config.param_dtype,
                                 reduce_dtype=dp_config.reduce_dtype)
            else:
                apply_generic_fsdp(model, dp_mesh, dp_config)
            model._fsdp_extra_dims = extra
            model._fsdp_enabled = True
            # the group the parameter shards are spread over (dp_shard under HSDP): squared gradient norms add up over it
            shard_dim = next((n for n in (MeshDimName.dp_shard, MeshDimName.dp) if n in names_), None)
            model._fsdp_shard_group = world_mesh[shard_dim].get_group() if (
                shard_dim is not None and world_mesh[shard_dim].size() > 1) else None
    if world_mesh is not None and ep_requested:
        # copies of one expert shard on ranks that read other batches (ep_size smaller than the data-parallel size)
        from .parallel.mesh import get_expert_replica_group

        model._expert_replica_group = get_expert_replica_group(world_mesh)
    if world_mesh is not None and not hasattr(model, "_replica_group"):
        # un-sharded data parallelism: gradients are averaged over the ranks that hold the same parameters
        model._replica_group = get_replica_group(world_mesh)
        if model._replica_group is not None and not getattr(model, "_fsdp_enabled", False):
            model._needs_grad_sync = True
    if device is not None and getattr(model, "_init_on_parallelize", False) and hasattr(model, "init_weights"):
        model.init_weights(device=device, world_mesh=world_mesh)
    return model
