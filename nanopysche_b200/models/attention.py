"""Multi-head / grouped-query attention (reference: model/attention.py:36-265).

Same constructor and parameter names as the reference (``w_q, w_k, w_v, w_out``, optional per-head
``q_norm``/``k_norm`` LayerNorms, RoPE, KV cache, TP and CP hooks). Differences by design:

* K/V are never expanded to the query head count; the attention op is GQA-native.
* On bf16 CUDA tensors the three projections run as one tcgen05 GEMM over a fused ``[q|k|v]``
  weight view (set up by ``optim.arena.ParamArena`` when the three weights are adjacent), and RoPE
  is applied in place on the q and k slices of its output.
* TP uses both Megatron operators (input-side backward all-reduce, output-side forward all-reduce);
  ``w_out`` is sliced on its input dimension by head count, not by ``shape[0]``.
* Under CP the rotary positions are the global positions of this rank's sequence shard.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn as nn

from ..ops import _lib
from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import rope as rope_ops
from .rope import RoPEScalingConfig, RotaryEmbedding
from .tp_utils import copy_to_tp_region, differentiable_all_reduce


class Attention(nn.Module):
    def __init__(self, *, d_model: int, n_heads: int, n_kv_heads: Optional[int] = None, bias: bool = False,
                 rope_base: float = 10000.0, max_seq_len: int = 8192, head_dim: Optional[int] = None,
                 qk_norm: bool = False, rope_head_first: bool = True,
                 rope_scaling: Optional[RoPEScalingConfig] = None, partial_rotary_factor: float = 1.0,
                 output_dropout: float = 0.0, dtype=None, device=None):
        super().__init__()
        self.d_model = d_model
        self.n_heads = n_heads
        self.n_kv_heads = n_kv_heads or n_heads
        assert n_heads % self.n_kv_heads == 0, "n_heads must be a multiple of n_kv_heads"
        self.head_dim = head_dim or d_model // n_heads
        self.n_rep = n_heads // self.n_kv_heads
        kw = dict(dtype=dtype, device=device)
        self.w_q = nn.Linear(d_model, n_heads * self.head_dim, bias=bias, **kw)
        self.w_k = nn.Linear(d_model, self.n_kv_heads * self.head_dim, bias=bias, **kw)
        self.w_v = nn.Linear(d_model, self.n_kv_heads * self.head_dim, bias=bias, **kw)
        self.w_out = nn.Linear(n_heads * self.head_dim, d_model, bias=bias, **kw)
        self.q_norm = nn.LayerNorm(self.head_dim, device=device) if qk_norm else None
        self.k_norm = nn.LayerNorm(self.head_dim, device=device) if qk_norm else None
        self.rope = RotaryEmbedding(self.head_dim, base=rope_base, max_seq_len=max_seq_len,
                                    head_first=rope_head_first, partial_rotary_factor=partial_rotary_factor,
                                    scaling=rope_scaling)
        # as in the reference (model/attention.py:81,109-110,186-187): dropout on the attention output *before* the
        # output projection, ``None`` when off; ``w_g`` is the reference's unused gate slot
        self.output_dropout = nn.Dropout(output_dropout) if output_dropout > 0 else None
        self.rope_head_first = rope_head_first
        self.w_g: Optional[nn.Linear] = None
        self._tp_size = 1
        self._tp_group = None
        self._cp_module = None
        self._local_heads = n_heads
        self._local_kv_heads = self.n_kv_heads
        self._fused_qkv: Optional[torch.Tensor] = None  # [q|k|v] weight view, set by the parameter arena
        self._tp_rt = None  # ops.tp_fused.TPRuntime when the fused sequence-parallel TP path is on

    # ------------------------------------------------------------------ forward
    def _project_qkv(self, x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        B, S, _ = x.shape
        hq, hkv, hd = self._local_heads, self._local_kv_heads, self.head_dim
        fused = self._fused_qkv
        if fused is not None and _lib.on(x) and x.dtype == fused.dtype and self.w_q.bias is None:
            qkv = gemm_ops.linear(x, fused)  # [B, S, (hq + 2 hkv) * hd]
            q = qkv[..., : hq * hd].unflatten(-1, (hq, hd))
            k = qkv[..., hq * hd:(hq + hkv) * hd].unflatten(-1, (hkv, hd))
            v = qkv[..., (hq + hkv) * hd:].unflatten(-1, (hkv, hd))
            return q, k, v
        q = gemm_ops.linear(x, self.w_q.weight, self.w_q.bias).view(B, S, hq, hd)
        k = gemm_ops.linear(x, self.w_k.weight, self.w_k.bias).view(B, S, hkv, hd)
        v = gemm_ops.linear(x, self.w_v.weight, self.w_v.bias).view(B, S, hkv, hd)
        return q, k, v

    def sdpa(self, q, k, v, *, causal: bool = True, attn_mask=None):
        """Attention on ``[B, S, H, hd]`` tensors (K/V with their own head count)."""
        return attn_ops.attention(q, k, v, causal=causal, attn_mask=attn_mask)

    def forward(self, x: torch.Tensor, *, causal: bool = True, attn_mask: Optional[torch.Tensor] = None,
                kv_cache: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, start_pos: int = 0,
                position_ids: Optional[torch.Tensor] = None, return_kv: bool = False, **_):
        from ..ops.tp_fused import active as _sp_active

        rt = self._tp_rt if _sp_active(self._tp_rt, x) else None
        hq, hkv, hd = self._local_heads, self._local_kv_heads, self.head_dim
        qkv = None  # fused projection output [B, S, (hq + 2 hkv) * hd] when one GEMM produced all three
        if rt is not None:
            # sequence-parallel input [1, M/tp, D]: all-gather fused into the QKV GEMM
            from ..ops import tp_fused

            B, S = rt.batch_shape
            w = self._fused_qkv if self._fused_qkv is not None else \
                torch.cat([self.w_q.weight, self.w_k.weight, self.w_v.weight], dim=0)
            qkv = tp_fused.ag_linear(x.reshape(-1, x.shape[-1]), w, rt).view(B, S, -1)
        else:
            B, S, _ = x.shape
            x = copy_to_tp_region(x, self._tp_group, self._tp_size)
            fused = self._fused_qkv
            if fused is not None and _lib.on(x) and x.dtype == fused.dtype and self.w_q.bias is None:
                qkv = gemm_ops.linear(x, fused)
        if position_ids is None and self._cp_module is not None:
            position_ids = self._cp_module.local_positions(S, x.device)
        max_pos = start_pos + S if position_ids is None else None
        if max_pos is None:
            max_pos = self._cp_module.global_seq_len(S) if self._cp_module is not None else \
                int(position_ids.max().item()) + 1
        cos, sin = self.rope.half_tables(max_pos, x.device)
        pid = None
        if position_ids is not None:
            pid = position_ids if position_ids.dim() == 2 else position_ids[None, :].expand(B, S)
        if qkv is not None and self.q_norm is None:
            q, k, v = rope_ops.qkv_rope(qkv, cos, sin, hq, hkv, hd, start_pos, pid)  # split + rotate in one kernel
        elif qkv is not None and self.q_norm.bias is not None and \
                rope_ops.qkv_norm_rope_supported(qkv, cos, hq, hkv, hd):
            # split + per-head LayerNorm of q and k + rotate in one kernel
            q, k, v = rope_ops.qkv_norm_rope(qkv, self.q_norm, self.k_norm, cos, sin, hq, hkv, start_pos, pid)
        else:
            if qkv is not None:
                q = qkv[..., : hq * hd].unflatten(-1, (hq, hd))
                k = qkv[..., hq * hd:(hq + hkv) * hd].unflatten(-1, (hkv, hd))
                v = qkv[..., (hq + hkv) * hd:].unflatten(-1, (hkv, hd))
            else:
                q, k, v = self._project_qkv(x)
            if self.q_norm is not None:
                q = self.q_norm(q.float()).to(x.dtype) if q.dtype != torch.float32 else self.q_norm(q)
                k = self.k_norm(k.float()).to(x.dtype) if k.dtype != torch.float32 else self.k_norm(k)
            q = rope_ops.apply_rope(q, cos, sin, start_pos, pid)
            k = rope_ops.apply_rope(k, cos, sin, start_pos, pid)
        if kv_cache is not None:
            k = torch.cat([kv_cache[0], k], dim=1)
            v = torch.cat([kv_cache[1], v], dim=1)
        if self._cp_module is not None:
            o = self._cp_module(q, k, v, causal=causal)
        else:
            o = self.sdpa(q, k, v, causal=causal, attn_mask=attn_mask)
        o = o.reshape(B, S, self._local_heads * self.head_dim)
        if self.output_dropout is not None:
            o = self.output_dropout(o)
        if rt is not None:
            from ..ops import tp_fused

            # GEMM -> reduce-scatter fused: back to the sequence shard [1, M/tp, D]
            out = tp_fused.linear_rs(o.reshape(B * S, -1), self.w_out.weight, rt).unsqueeze(0)
        else:
            out = gemm_ops.linear(o, self.w_out.weight, None)
            out = differentiable_all_reduce(out, self._tp_group, self._tp_size)
        if self.w_out.bias is not None:
            out = out + self.w_out.bias
        if return_kv:
            return out, (k, v)
        return out

    # ------------------------------------------------------------------ parallel hooks
    def apply_tp(self, tp_mesh, **_):
        """Shard heads over the TP mesh: q/k/v column-wise, w_out row-wise (by input features)."""
        group = tp_mesh.get_group() if hasattr(tp_mesh, "get_group") else tp_mesh
        import torch.distributed as dist

        tp = dist.get_world_size(group)
        rank = dist.get_rank(group)
        if tp <= 1:
            return
        assert self.n_heads % tp == 0 and self.n_kv_heads % tp == 0, "heads must divide the TP degree"
        self._tp_size, self._tp_group = tp, group
        self._local_heads = self.n_heads // tp
        self._local_kv_heads = self.n_kv_heads // tp
        hd = self.head_dim

        def col(lin: nn.Linear, heads_local: int):
            w = lin.weight.data.view(tp, heads_local * hd, lin.in_features)[rank].clone()
            lin.weight = nn.Parameter(w)
            if lin.bias is not None:
                lin.bias = nn.Parameter(lin.bias.data.view(tp, -1)[rank].clone())
            lin.out_features = heads_local * hd

        col(self.w_q, self._local_heads)
        col(self.w_k, self._local_kv_heads)
        col(self.w_v, self._local_kv_heads)
        n_in = self._local_heads * hd
        self.w_out.weight = nn.Parameter(self.w_out.weight.data[:, rank * n_in:(rank + 1) * n_in].clone())
        self.w_out.in_features = n_in
        self._fused_qkv = None
        for lin in (self.w_q, self.w_k, self.w_v, self.w_out):   # shards differ between TP peers: never averaged
            lin.weight._tp_sharded = group                       # over them, and their norms add up over them
            if lin.bias is not None and lin is not self.w_out:
                lin.bias._tp_sharded = group

    def apply_cp(self, cp_mesh, *, ring=None, uly=None, **_):
        """Route attention through the context-parallel module (ring by default, Ulysses if ``uly``)."""
        from ..parallel.context_parallel import RingAttention

        group = cp_mesh.get_group() if hasattr(cp_mesh, "get_group") else cp_mesh
        use_ulysses = bool(uly) and not bool(ring)
        self._cp_module = RingAttention(group, use_ulysses=use_ulysses, use_zigzag=True)
