"""Model factories (reference: model_factory.py:38-177).

``build_model(ctx, factory_spec=None)`` returns ``(model, optimizer | None, scheduler | None)``: the
default Transformer for the CLI presets, or the result of a user ``"module.path:callable"`` factory
(which may return a model or a ``(model, opt[, sched])`` tuple and gets the generic parallel hooks).
``convert_to_moe`` generalises the reference's ``apply_moe_hybrid`` (MoE on even layers, expert
hidden = dense hidden, no dense FFN): interval / offset / expert hidden / capacity / keeping the
dense FFN are arguments, so "MoE in every layer" and "dense on even, MoE on odd" are both expressible.
"""
from __future__ import annotations

import importlib
from dataclasses import dataclass
from typing import Any, Callable, Optional

import torch
import torch.nn as nn

from .models.feed_forward import FeedForward
from .models.moe import MoEBase
from .models.parallel_adapter import ensure_parallel_hooks
from .models.transformer import Transformer, TransformerBlock


@dataclass
class ModelBuildContext:
    vocab_size: int = 32000
    seq_len: int = 2048
    device: Any = "cpu"
    model_preset: str = "125m"
    preset: Optional[dict] = None
    use_moe: bool = False
    num_experts: int = 8
    moe_top_k: int = 2
    fp8_recipe: str = "none"
    dtype: torch.dtype = torch.float32
    fp8_gemm_threshold: int = 1000000
    moe_interval: int = 2
    moe_offset: int = 0
    moe_hidden: Optional[int] = None
    moe_capacity_factor: Optional[float] = None
    moe_keep_dense_ffn: bool = False


def load_factory(spec: str) -> Callable:
    """``"package.module:callable"`` -> the callable."""
    if ":" not in spec:
        raise ValueError(f"factory spec must look like 'module.path:callable', got {spec!r}")
    mod, attr = spec.split(":", 1)
    fn = getattr(importlib.import_module(mod), attr, None)
    if not callable(fn):
        raise ValueError(f"{spec!r} does not name a callable")
    return fn


def build_default_transformer(ctx: ModelBuildContext) -> Transformer:
    from .config import TransformerConfig

    p = dict(ctx.preset or {})
    cfg = TransformerConfig(vocab_size=ctx.vocab_size, d_model=p.get("d_model", 768), n_layers=p.get("n_layers", 12),
                            n_heads=p.get("n_heads", 12), n_kv_heads=p.get("n_kv_heads", p.get("n_heads", 12)),
                            ffn_hidden=p.get("ffn_hidden"), rope_base=p.get("rope_base", 500000.0),
                            max_seq_len=ctx.seq_len, qk_norm=p.get("qk_norm", True))
    return cfg.build(dtype=ctx.dtype, init_device=str(ctx.device) if str(ctx.device) != "cuda" else "cuda")


def convert_to_moe(model: Transformer, *, num_experts: int, top_k: int, hidden: Optional[int] = None,
                   interval: int = 2, offset: int = 0, capacity_factor: Optional[float] = None,
                   keep_dense_ffn: bool = False, fp8_flow_moe: bool = False, fp8_recipe: str = "none",
                   fp8_gemm_threshold: int = 1000000, dtype=None, **moe_kwargs) -> Transformer:
    for idx in range(model.n_layers):
        key = str(idx)
        if key not in model.blocks or idx % max(interval, 1) != offset % max(interval, 1):
            continue
        blk = model.blocks[key]
        if not isinstance(blk, TransformerBlock):
            continue
        dense = blk.feed_forward if isinstance(blk.feed_forward, FeedForward) else None
        h = hidden or (dense.hidden_size if dense is not None else None)
        dev = next(blk.parameters()).device
        moe = MoEBase(d_model=model.d_model, hidden_size=h, num_experts=num_experts, top_k=top_k,
                      capacity_factor=capacity_factor, fp8_flow_moe=fp8_flow_moe and fp8_recipe != "none",
                      fp8_recipe=fp8_recipe, fp8_gemm_threshold=fp8_gemm_threshold,
                      dtype=dtype or next(blk.parameters()).dtype, device=dev, **moe_kwargs)
        model.replace_block_with_moe_hybrid(idx, moe, dense_ffn=dense if keep_dense_ffn else None)
    return model


def apply_moe_hybrid(model: Transformer, ctx: ModelBuildContext) -> Transformer:
    """The CLI's ``--use-moe`` conversion (defaults: MoE on even layers, expert hidden = dense hidden)."""
    return convert_to_moe(model, num_experts=ctx.num_experts, top_k=ctx.moe_top_k, hidden=ctx.moe_hidden,
                          interval=ctx.moe_interval, offset=ctx.moe_offset,
                          capacity_factor=ctx.moe_capacity_factor, keep_dense_ffn=ctx.moe_keep_dense_ffn,
                          fp8_flow_moe=ctx.fp8_recipe != "none", fp8_recipe=ctx.fp8_recipe,
                          fp8_gemm_threshold=ctx.fp8_gemm_threshold, dtype=ctx.dtype)


def build_model(ctx: ModelBuildContext, factory_spec: Optional[str] = None):
    if factory_spec:
        res = load_factory(factory_spec)(ctx)
        opt = sched = None
        if isinstance(res, tuple):
            model = res[0]
            opt = res[1] if len(res) > 1 else None
            sched = res[2] if len(res) > 2 else None
        else:
            model = res
        if not isinstance(model, nn.Module):
            raise TypeError("model factory must return an nn.Module (or a tuple starting with one)")
        return ensure_parallel_hooks(model), opt, sched
    model = build_default_transformer(ctx)
    if ctx.use_moe:
        apply_moe_hybrid(model, ctx)
    return model, None, None
