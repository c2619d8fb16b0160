"""Model protocol helpers (reference: model/protocol.py:18-91): which parallel hooks a model offers."""
from __future__ import annotations

import warnings

from typing import Optional

import torch.nn as nn

PARALLEL_HOOKS = ("apply_pp", "apply_tp", "apply_cp", "apply_ep", "apply_fsdp", "apply_compile", "init_weights")
MOE_HOOKS = ("replace_block_with_moe_hybrid",)
_HOOK_OF = {"pp": "apply_pp", "tp": "apply_tp", "cp": "apply_cp", "ep": "apply_ep", "fsdp": "apply_fsdp",
            "compile": "apply_compile"}


def has_hook(model: nn.Module, name: str) -> bool:
    return callable(getattr(model, name, None))


def model_display_name(model: nn.Module, preset: Optional[str] = None) -> str:
    """The preset's name when the model came from one, else the class name (reference: model/protocol.py:75-78)."""
    return preset or type(model).__name__


def unsupported_parallelism(model: nn.Module, *, tp: int = 1, pp: int = 1, cp: int = 1, ep: int = 1,
                            fsdp: bool = False, compile: bool = False, compile_model: bool = False) -> list[str]:
    """Names of the requested parallelism kinds the model has no hook for. Degrees (``tp=2``) or the reference's
    booleans (``tp=True``, ``compile_model=True``; model/protocol.py) are both accepted."""
    def on(v):
        return v is True or (not isinstance(v, bool) and v > 1)

    wanted = {"tp": on(tp), "pp": on(pp), "cp": on(cp), "ep": on(ep), "fsdp": bool(fsdp),
              "compile": bool(compile or compile_model)}
    return [k for k, on in wanted.items() if on and not has_hook(model, _HOOK_OF[k])]


def warn_unsupported_parallelism(model: nn.Module, missing=None, **kw) -> list[str]:
    """Warns about the parallel modes in ``missing`` (the reference's form, model/protocol.py:61-72); without a list
    the modes asked for by keyword (``tp=2, pp=2, ...``) are checked against the model's hooks first."""
    if missing is None:
        missing = unsupported_parallelism(model, **kw)
    missing = list(missing)
    if missing:
        warnings.warn(f"{model_display_name(model)} has no hook for: {', '.join(missing)}; those are skipped")
    return missing


def count_parameters(model: nn.Module, trainable_only: bool = False) -> dict:
    """``{"num_params", "num_non_embed_params"}`` (reference: model/protocol.py:81-91); the embedding is looked up as
    ``model.embeddings`` or ``model.embed``."""
    num = sum(p.numel() for p in model.parameters() if p.requires_grad or not trainable_only)
    emb = 0
    for name in ("embeddings", "embed"):
        w = getattr(getattr(model, name, None), "weight", None)
        if w is not None and (w.requires_grad or not trainable_only):
            emb = w.numel()
            break
    return {"num_params": num, "num_non_embed_params": num - emb}
