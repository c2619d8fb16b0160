"""Dataclass configuration system (reference: config.py:42-329).

``Config`` gives every config JSON / YAML / TOML round-trips, nested ``_from_dict``, dotted-path
``merge`` and a generic ``from_cli``; ``TransformerConfig.build()`` / ``TrainingConfig.build()`` /
``ExperimentConfig.build()`` assemble model, optimizer, scheduler and the runtime training config.
``TrainingConfig.build`` forwards the schedule fields and ``log_interval`` that the reference drops,
and ``TransformerConfig`` can place MoE layers (``moe_interval`` / ``moe_offset`` / expert hidden
size / capacity factor / DeepSeek-V3 bias rate / shared expert / jitter) and use GQA, which the 1B
and 7B mixture-of-experts configurations (GQA trunks, MoE in every or every other layer) need.
"""
from __future__ import annotations

import copy
import dataclasses
import json
import typing
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Any, Dict, Optional

try:
    import yaml as _yaml
    _HAS_YAML = True
except ImportError:  # pragma: no cover
    _HAS_YAML = False
try:
    import tomllib
except ImportError:  # pragma: no cover
    tomllib = None
try:
    import tomli_w as _tomli_w
    _HAS_TOMLI_W = True
except ImportError:
    _HAS_TOMLI_W = False


def _coerce(value: str) -> Any:
    try:
        return int(value)
    except ValueError:
        pass
    try:
        return float(value)
    except ValueError:
        pass
    low = value.lower()
    if low in ("true", "false"):
        return low == "true"
    if low in ("none", "null"):
        return None
    return value


@dataclass
class Config:
    def build(self, **kwargs):
        raise NotImplementedError

    def as_dict(self) -> Dict[str, Any]:
        return asdict(self)

    def save(self, path):
        path = Path(path)
        path.parent.mkdir(parents=True, exist_ok=True)
        data = self.as_dict()
        if path.suffix == ".toml":
            if not _HAS_TOMLI_W:
                raise ImportError("tomli_w is required for TOML output")
            with open(path, "wb") as f:
                _tomli_w.dump(data, f)
            return
        with open(path, "w") as f:
            if path.suffix in (".yaml", ".yml") and _HAS_YAML:
                _yaml.safe_dump(data, f, default_flow_style=False)
            else:
                json.dump(data, f, indent=2, default=str)

    @classmethod
    def load(cls, path):
        path = Path(path)
        if path.suffix == ".toml":
            if tomllib is None:
                raise ImportError("TOML support requires Python 3.11+")
            with open(path, "rb") as f:
                data = tomllib.load(f)
        elif path.suffix in (".yaml", ".yml") and _HAS_YAML:
            with open(path) as f:
                data = _yaml.safe_load(f)
        else:
            with open(path) as f:
                data = json.load(f)
        return cls._from_dict(data or {})

    @classmethod
    def _from_dict(cls, data: Dict[str, Any]):
        try:
            hints = typing.get_type_hints(cls)
        except Exception:  # noqa: BLE001
            hints = {}
        kwargs = {}
        for f in dataclasses.fields(cls):
            if f.name not in data:
                continue
            t, v = hints.get(f.name, f.type), data[f.name]
            if isinstance(v, dict) and isinstance(t, type) and issubclass(t, Config):
                kwargs[f.name] = t._from_dict(v)
            else:
                kwargs[f.name] = v
        return cls(**kwargs)

    def merge(self, overrides: Dict[str, Any]):
        obj = copy.deepcopy(self)
        for key, value in overrides.items():
            parts = key.split(".")
            cur = obj
            ok = True
            for p in parts[:-1]:
                if hasattr(cur, p):
                    cur = getattr(cur, p)
                else:
                    ok = False
                    break
            if ok and hasattr(cur, parts[-1]):
                setattr(cur, parts[-1], value)
        return obj

    @classmethod
    def from_cli(cls, args: list):
        overrides, i = {}, 0
        while i < len(args):
            if args[i].startswith("--") and i + 1 < len(args):
                overrides[args[i][2:]] = _coerce(args[i + 1])
                i += 2
            else:
                i += 1
        return cls().merge(overrides)


@dataclass
class TransformerConfig(Config):
    vocab_size: int = 32000
    d_model: int = 4096
    n_layers: int = 32
    n_heads: int = 32
    n_kv_heads: Optional[int] = None
    head_dim: Optional[int] = None
    rope_base: float = 500000.0
    max_seq_len: int = 8192
    qk_norm: bool = True
    ffn_hidden: Optional[int] = None
    use_moe: bool = False
    num_experts: int = 8
    moe_top_k: int = 2
    tie_word_embeddings: bool = False
    dropout: float = 0.0
    fp8_flow_moe: bool = False
    fp8_recipe: str = "none"
    fp8_gemm_threshold: int = 1000000
    tp_size: int = 1
    pp_size: int = 1
    cp_size: int = 1
    dp_size: int = 1
    fsdp_wrapping: str = "full"
    fsdp_mixed_precision: Optional[str] = "bf16"
    activation_checkpointing: Optional[str] = None
    checkpoint_interval: Optional[int] = None
    compile: bool = False
    # MoE placement (beyond the reference): layer i is MoE when i % moe_interval == moe_offset
    moe_interval: int = 2
    moe_offset: int = 0
    moe_hidden: Optional[int] = None
    moe_capacity_factor: Optional[float] = None
    moe_keep_dense_ffn: bool = False
    moe_bias_gamma: Optional[float] = None      # DeepSeek-V3 auxiliary-loss-free balancing: bias update rate
    moe_shared_expert: bool = False
    moe_jitter_eps: Optional[float] = None
    moe_z_loss: Optional[float] = None
    rope_scaling_factor: float = 1.0
    rope_scaling_type: str = "piecewise"
    dtype: str = "float32"
    init_std: Optional[float] = None
    xent_chunk_rows: int = 0     # > 0: head projection + loss over this many rows at a time (full logits never formed)

    def build(self, **kwargs):
        import torch

        from .models.rope import RoPEScalingConfig
        from .models.transformer import Transformer

        n_kv = self.n_kv_heads or self.n_heads
        ffn = self.ffn_hidden or int(8 / 3 * self.d_model)
        ffn = ((ffn + 255) // 256) * 256
        scaling = None
        if self.rope_scaling_factor > 1.0:
            scaling = RoPEScalingConfig(factor=self.rope_scaling_factor, rope_type=self.rope_scaling_type,
                                        original_max_position_embeddings=self.max_seq_len)
        block = dict(n_heads=self.n_heads, n_kv_heads=n_kv, head_dim=self.head_dim, rope_base=self.rope_base,
                     max_seq_len=self.max_seq_len, qk_norm=self.qk_norm, ffn_hidden=ffn, dropout=self.dropout,
                     rope_scaling=scaling)
        block.update(kwargs.pop("block", {}))
        dtype = kwargs.pop("dtype", getattr(torch, self.dtype))
        model = Transformer(vocab_size=self.vocab_size, d_model=self.d_model, n_layers=self.n_layers, block=block,
                            tie_word_embeddings=self.tie_word_embeddings, dtype=dtype, **kwargs)
        if self.use_moe:
            from .model_factory import convert_to_moe

            convert_to_moe(model, num_experts=self.num_experts, top_k=self.moe_top_k,
                           hidden=self.moe_hidden or ffn, interval=self.moe_interval, offset=self.moe_offset,
                           capacity_factor=self.moe_capacity_factor, keep_dense_ffn=self.moe_keep_dense_ffn,
                           fp8_flow_moe=self.fp8_flow_moe, fp8_recipe=self.fp8_recipe,
                           fp8_gemm_threshold=self.fp8_gemm_threshold, dtype=dtype,
                           bias_gamma=self.moe_bias_gamma, shared_expert=self.moe_shared_expert,
                           jitter_eps=self.moe_jitter_eps, z_loss_multiplier=self.moe_z_loss)
        if self.init_std is not None:
            model.init_weights(std=self.init_std)
        model.loss_chunk_rows = int(self.xent_chunk_rows or 0)
        return model


@dataclass
class TrainingConfig(Config):
    global_batch_size: int = 1024
    micro_batch_size: int = 4
    sequence_length: int = 2048
    learning_rate: float = 3e-4
    min_lr: float = 3e-5
    weight_decay: float = 0.1
    max_grad_norm: float = 1.0
    warmup_steps: int = 2000
    max_steps: int = 600000
    schedule: str = "cosine"
    stable_steps: int = 0
    decay_steps: int = 0
    dtype: str = "bfloat16"
    save_interval: int = 1000
    save_dir: str = "checkpoints"
    log_interval: int = 10

    def build(self, **kwargs):
        import torch

        from .train.trainer import TrainingConfig as TC

        return TC(global_batch_size=self.global_batch_size, micro_batch_size=self.micro_batch_size,
                  sequence_length=self.sequence_length, learning_rate=self.learning_rate, min_lr=self.min_lr,
                  weight_decay=self.weight_decay, max_grad_norm=self.max_grad_norm, warmup_steps=self.warmup_steps,
                  max_steps=self.max_steps, dtype=getattr(torch, self.dtype), save_interval=self.save_interval,
                  save_dir=self.save_dir, log_interval=self.log_interval, **kwargs)

    def build_scheduler(self, optimizer):
        from .train.scheduler import CosineWithWarmup, WarmupStableDecay

        ratio = self.min_lr / self.learning_rate if self.learning_rate else 0.1
        if self.schedule == "wsd":
            return WarmupStableDecay(optimizer, self.warmup_steps, self.stable_steps, self.decay_steps, ratio)
        return CosineWithWarmup(optimizer, warmup_steps=self.warmup_steps, max_steps=self.max_steps,
                                min_lr_ratio=ratio)


@dataclass
class ExperimentConfig(Config):
    name: str = "experiment"
    model: TransformerConfig = field(default_factory=TransformerConfig)
    training: TrainingConfig = field(default_factory=TrainingConfig)
    seed: int = 42
    model_factory: Optional[str] = None

    def build(self, **kwargs):
        import torch

        from .model_factory import ModelBuildContext, build_model

        optimizer = scheduler = None
        if self.model_factory:
            ctx = ModelBuildContext(vocab_size=self.model.vocab_size, seq_len=self.model.max_seq_len,
                                    device=kwargs.get("device", "cpu"), model_preset="custom", preset=None,
                                    use_moe=self.model.use_moe, num_experts=self.model.num_experts,
                                    moe_top_k=self.model.moe_top_k, fp8_recipe=self.model.fp8_recipe,
                                    fp8_gemm_threshold=self.model.fp8_gemm_threshold,
                                    dtype=kwargs.get("dtype", torch.float32))
            model, optimizer, scheduler = build_model(ctx, factory_spec=self.model_factory)
        else:
            model = self.model.build()
        if optimizer is None:
            optimizer = torch.optim.AdamW(model.parameters(), lr=self.training.learning_rate,
                                          weight_decay=self.training.weight_decay, betas=(0.9, 0.95))
        if scheduler is None:
            scheduler = self.training.build_scheduler(optimizer)
        return model, optimizer, scheduler, self.training.build()
