"""Tensor-parallel configuration and the sequence-parallel layout helper
(reference: distributed/tensor_parallel.py:29-85).

``TensorParallelConfig.enable_async`` selects the fused all-gather->GEMM / GEMM->reduce-scatter
kernels (``ops/tp_fused.py``) instead of separate collectives; the reference's flag only toggled an
inductor micro-pipelining option that its manual TP never used.
"""
from __future__ import annotations

from dataclasses import dataclass

from typing import Optional

import torch.nn as nn

from ..models.tp_utils import gather_seq, scatter_seq


@dataclass
class TensorParallelConfig:
    degree: int = 1
    enable_async: bool = False
    sequence_parallel: bool = False

    def maybe_enable_async_tp(self, tp_mesh=None) -> bool:
        """Returns True when the fused TP kernels are switched on for this mesh."""
        if not self.enable_async or tp_mesh is None or self.degree <= 1:
            return False
        from . import symm

        return symm.available()


class SequenceParallel(nn.Module):
    """Wraps a module that works on sequence shards (norms, dropout): gathers the full sequence on
    exit (``gather_output``) or scatters on entry (``scatter_input``) over the TP group, along
    ``sequence_dim``; the conjugate collective runs in backward."""

    def __init__(self, module: Optional[nn.Module] = None, tp_group=None, tp_size: int = 1, *, sequence_dim: int = 1,
                 gather_output: bool = True, scatter_input: bool = False, use_local_output: bool = False,
                 output_layouts=None):
        """``use_local_output`` / ``output_layouts`` belong to the reference's DTensor style object
        (distributed/tensor_parallel.py), which has no module argument; they are accepted so that its keyword form
        constructs, and ``module`` may then be given later (``.module = ...``). Tensors here are plain local tensors."""
        super().__init__()
        self.use_local_output, self.output_layouts = use_local_output, output_layouts
        self.module = module if module is not None else nn.Identity()
        self.tp_group, self.tp_size = tp_group, tp_size
        self.sequence_dim = sequence_dim
        self.gather_output, self.scatter_input = gather_output, scatter_input

    def forward(self, x, *a, **k):
        if self.scatter_input:
            x = scatter_seq(x, self.tp_group, self.tp_size, self.sequence_dim)
        y = self.module(x, *a, **k)
        if self.gather_output:
            y = gather_seq(y, self.tp_group, self.tp_size, self.sequence_dim)
        return y
