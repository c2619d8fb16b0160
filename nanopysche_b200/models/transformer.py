"""Decoder blocks and the Transformer (reference: model/transformer.py:38-651).

Same constructor signatures, module / parameter names (= checkpoint keys) and hook methods as the
reference. Differences by design:

* ``Transformer.forward`` is pipeline-stage aware: a stage without embeddings takes hidden states,
  a stage without a head returns them (the reference unpacks ``input_ids.shape`` unconditionally).
* The loss is computed over all positions against labels shifted by one with the last position
  ignored - identical to ``CE(logits[:, :-1], labels[:, 1:])`` without the slice copy - through the
  fused cross-entropy op; the auxiliary loss stays a device tensor (no ``.item()`` per forward).
* ``MoEHybridTransformerBlock`` overlaps for real: the dense FFN runs on a side stream while the
  dispatch / expert / combine kernels run on the main one.
* The second norm of a block is fused with the residual add in front of it.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn

from ..ops import _lib
from ..ops import embedding as embedding_ops
from ..ops import gemm as gemm_ops
from ..ops import xent as xent_ops
from .attention import Attention
from .feed_forward import FeedForward
from .moe import ExpertParallelConfig, MoEBase
from .norm import RMSNorm


class TransformerBlock(nn.Module):
    def __init__(self, *, d_model: int, block_idx: int = 0, n_layers: int = 1, n_heads: int = 32,
                 n_kv_heads: Optional[int] = None, head_dim: Optional[int] = None, rope_base: float = 10000.0,
                 max_seq_len: int = 8192, qk_norm: bool = False, ffn_hidden: Optional[int] = None,
                 attention: Optional[Attention] = None, feed_forward: Optional[nn.Module] = None,
                 attention_norm: Optional[RMSNorm] = None, feed_forward_norm: Optional[RMSNorm] = None,
                 dropout: float = 0.0, rope_scaling=None, dtype=None, device=None):
        super().__init__()
        self.d_model = d_model
        self.block_idx = block_idx
        self.attention_norm = attention_norm or RMSNorm(d_model, device=device)
        self.attention = attention if attention is not None else Attention(
            d_model=d_model, n_heads=n_heads, n_kv_heads=n_kv_heads, head_dim=head_dim, rope_base=rope_base,
            max_seq_len=max_seq_len, qk_norm=qk_norm, rope_scaling=rope_scaling, dtype=dtype, device=device)
        self.feed_forward_norm = feed_forward_norm or RMSNorm(d_model, device=device)
        self.feed_forward = feed_forward if feed_forward is not None else FeedForward(
            d_model=d_model, hidden_size=ffn_hidden, dtype=dtype, device=device)
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    def forward(self, x: torch.Tensor, *, causal: bool = True, attn_mask: Optional[torch.Tensor] = None, **kwargs):
        a = self.dropout(self.attention(self.attention_norm(x), causal=causal, attn_mask=attn_mask, **kwargs))
        y, h = self.feed_forward_norm(a, residual=x)
        return h + self.dropout(self.feed_forward(y))

    def apply_tp(self, tp_mesh, *, sequence_parallel: bool = False):
        self.attention.apply_tp(tp_mesh)
        if hasattr(self.feed_forward, "apply_tp"):
            self.feed_forward.apply_tp(tp_mesh)

    def apply_cp(self, cp_mesh, *, ring=None, uly=None):
        self.attention.apply_cp(cp_mesh, ring=ring, uly=uly)

    def apply_fsdp(self, dp_mesh=None, *, wrapping_strategy="full", reshard_after_forward=True, mp_policy=None,
                   prefetch_factor: int = 0, **kw):
        from ..parallel.fsdp import shard_module

        if str(getattr(wrapping_strategy, "value", wrapping_strategy)) == "fine_grained":
            shard_module(self.attention, dp_mesh, reshard_after_forward=reshard_after_forward, mp_policy=mp_policy)
            shard_module(self.feed_forward, dp_mesh, reshard_after_forward=reshard_after_forward,
                         mp_policy=mp_policy)
        shard_module(self, dp_mesh, reshard_after_forward=reshard_after_forward, mp_policy=mp_policy)


class MoEHybridTransformerBlock(nn.Module):
    """Attention + (optional dense FFN) + MoE: ``x = h + dense(h) + moe(h)`` with ``h = x + attn(x)``."""

    def __init__(self, *, d_model: int, block_idx: int = 0, n_layers: int = 1, attention: Attention, moe: MoEBase,
                 dense_ffn: Optional[FeedForward] = None, attention_norm: Optional[RMSNorm] = None,
                 moe_norm: Optional[RMSNorm] = None, dense_norm: Optional[RMSNorm] = None, dropout: float = 0.0):
        super().__init__()
        self.d_model = d_model
        self.block_idx = block_idx
        self.attention_norm = attention_norm or RMSNorm(d_model)
        self.attention = attention
        self.moe = moe
        self.moe_norm = moe_norm or RMSNorm(d_model)
        self.dense_ffn = dense_ffn
        self.dense_norm = (dense_norm or RMSNorm(d_model)) if dense_ffn is not None else None
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()
        self._side_stream: Optional[torch.cuda.Stream] = None

    def forward(self, x: torch.Tensor, *, causal: bool = True, attn_mask: Optional[torch.Tensor] = None, **kwargs):
        B, S, D = x.shape
        a = self.dropout(self.attention(self.attention_norm(x), causal=causal, attn_mask=attn_mask, **kwargs))
        y, h = self.moe_norm(a, residual=x)
        dense_out = None
        overlap = self.dense_ffn is not None and x.is_cuda and not torch.cuda.is_current_stream_capturing()
        if overlap:
            # dense FFN on a side stream while dispatch -> experts -> combine run on the main stream
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream()
            side, main = self._side_stream, torch.cuda.current_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                dense_out = self.dense_ffn(self.dense_norm(h))
        if self.moe._can_fuse(y):
            moe_out = self.moe(y)
        else:
            x_flat, w_flat, i_flat, aux, dropped, keep_mask = self.moe.route(y)
            local_x, local_w, local_i, meta = self.moe.dispatch(x_flat, i_flat, w_flat)
            if self.dense_ffn is not None and not overlap:
                dense_out = self.dense_ffn(self.dense_norm(h))
            expert_out = self.moe.local_compute(local_x, local_w, local_i)
            moe_flat = self.moe.combine(expert_out, meta, x_flat, w_flat, i_flat)
            moe_out = self.moe.reassemble(moe_flat, dropped=dropped, keep_mask=keep_mask, B=B, S=S, D=D)
        if self.dense_ffn is not None and dense_out is None:
            dense_out = self.dense_ffn(self.dense_norm(h))
        if overlap:
            torch.cuda.current_stream().wait_stream(self._side_stream)
            dense_out.record_stream(torch.cuda.current_stream())
        out = h + moe_out
        if dense_out is not None:
            out = out + dense_out
        return out

    @property
    def feed_forward(self) -> MoEBase:
        return self.moe

    def apply_tp(self, tp_mesh, **_):
        self.attention.apply_tp(tp_mesh)
        if self.dense_ffn is not None:
            self.dense_ffn.apply_tp(tp_mesh)

    def apply_cp(self, cp_mesh, *, ring=None, uly=None):
        self.attention.apply_cp(cp_mesh, ring=ring, uly=uly)

    def apply_fsdp(self, dp_mesh=None, *, wrapping_strategy="full", reshard_after_forward=True, mp_policy=None,
                   prefetch_factor: int = 0, **kw):
        from ..parallel.fsdp import shard_module

        shard_module(self, dp_mesh, reshard_after_forward=reshard_after_forward, mp_policy=mp_policy)


class Transformer(nn.Module):
    def __init__(self, *, d_model: int, vocab_size: int, n_layers: int, block: Optional[Dict[str, object]] = None,
                 lm_head: Optional[nn.Linear] = None, embedding_norm: Optional[RMSNorm] = None,
                 dtype: torch.dtype = torch.float32, init_device: str = "cpu", tie_word_embeddings: bool = False):
        super().__init__()
        self.d_model = d_model
        self.vocab_size = vocab_size
        self.n_layers = n_layers
        self.dtype = dtype
        self.embeddings = nn.Embedding(vocab_size, d_model, dtype=dtype, device=init_device)
        self.embedding_norm = embedding_norm
        self.blocks = nn.ModuleDict()
        for block_idx in range(n_layers):
            cfg = dict(block or {})
            cfg.setdefault("dtype", dtype)
            cfg.setdefault("device", init_device)
            self.blocks[str(block_idx)] = TransformerBlock(d_model=d_model, block_idx=block_idx, n_layers=n_layers,
                                                           **cfg)
        self.final_norm: Optional[RMSNorm] = None
        self.lm_head = lm_head or nn.Linear(d_model, vocab_size, bias=False, dtype=dtype, device=init_device)
        self.tie_word_embeddings = tie_word_embeddings
        if tie_word_embeddings:
            self.lm_head = None
        self._pp_enabled = False
        self._tp_enabled = False
        self._fsdp_enabled = False
        self._compile_enabled = False
        self._cp_group = None
        self._is_first_stage = True
        self._is_last_stage = True
        # > 0: with labels given, head projection and loss run together over this many rows at a time
        # (``ops.xent.linear_cross_entropy``); the full logits are then never formed and ``"logits"`` is None
        self.loss_chunk_rows = 0

    @property
    def num_params(self) -> int:
        return sum(p.numel() for p in self.parameters())

    @property
    def num_non_embedding_params(self) -> int:
        n = self.num_params
        if self.embeddings is not None:
            n -= self.embeddings.weight.numel()
        return n

    # ------------------------------------------------------------------ forward
    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None, *,
                labels_shifted: bool = False, return_logits: bool = True, **kwargs):
        """Returns ``{"logits", "loss"}`` plus ``"aux_loss"`` when MoE layers produced one (a stage without a head returns
        hidden states)."""
        if self.embeddings is not None and not input_ids.is_floating_point():
            emb = self.embeddings
            if type(emb) is nn.Embedding and emb.padding_idx is None and emb.max_norm is None and \
                    not self._fsdp_enabled and hasattr(emb.weight, "main_grad"):
                x = embedding_ops.embedding(input_ids, emb.weight)   # backward adds into the gradient arena
            else:
                x = emb(input_ids)
            if self.embedding_norm is not None:
                x = self.embedding_norm(x)
        else:
            x = input_ids  # hidden states from the previous pipeline stage
        tp_rt = None
        # every pipeline stage takes its row shard of the (replicated) hidden states it receives and hands the next
        # stage replicated rows again: the slice's backward leaves the other ranks' rows zero and the gather's backward
        # of the previous stage takes exactly this rank's rows, so the partial gradients never need a reduction
        if getattr(self, "_tp_fused", False) and x.dim() == 3 and \
                (getattr(self, "_tp_host", False) or (x.is_cuda and x.dtype == torch.bfloat16)):
            B0, S0, D0 = x.shape
            tp_rt = self._ensure_tp_runtime(B0, S0, x.device)
            x = x.reshape(B0 * S0, D0)[tp_rt.rank * tp_rt.Ms:(tp_rt.rank + 1) * tp_rt.Ms].unsqueeze(0)
        for name, blk in self.blocks.items():
            with _lib.nvtx_range("block." + name):
                x = blk(x, **kwargs)
        if tp_rt is not None:
            from ..ops.tp_fused import gather_rows_replicated

            x = gather_rows_replicated(x.reshape(tp_rt.Ms, -1), self._tp_group).view(B0, S0, -1)
        aux = self._collect_aux(x)
        if not self._is_last_stage or (self.lm_head is None and not self.tie_word_embeddings):
            return self._with_aux({"hidden_states": x}, aux)
        if self.final_norm is not None:
            x = self.final_norm(x)
        if labels is not None and getattr(self, "loss_chunk_rows", 0) > 0:
            w = self.lm_head.weight if self.lm_head is not None else self.embeddings.weight
            # a head weight that is sharded, quantised or wrapped takes the ordinary path below
            plain_head = not (self._fsdp_enabled and self.lm_head is not None) and \
                (self.lm_head is None or self.lm_head.bias is None) and type(w).__name__ != "DTensor" and \
                not any(hasattr(w, a) for a in ("_fsdp_rt", "_fp8_recipe", "_tp_sharded"))
            if plain_head:
                tgt = self._shift_labels(labels, labels_shifted)
                local = xent_ops.linear_cross_entropy(x.reshape(-1, x.shape[-1]), w, tgt.reshape(-1),
                                                      ignore_index=-100, chunk_rows=self.loss_chunk_rows)
                return self._with_aux({"logits": None, "loss": self._loss_over_cp_group(local, tgt)}, aux)
        if self._fsdp_enabled and self.lm_head is not None:
            logits = self.lm_head(x)  # through the module so its FSDP unshard hook runs
        else:
            w = self.lm_head.weight if self.lm_head is not None else self.embeddings.weight
            logits = gemm_ops.linear(x, w)
        out = self._with_aux({"logits": logits if return_logits else None}, aux)
        if labels is not None:
            out["loss"] = self.loss_from_logits(logits, labels, labels_shifted=labels_shifted)
        return out

    @staticmethod
    def _with_aux(out: dict, aux):
        """``"aux_loss"`` is present only when a MoE layer produced one, as in the reference
        (model/transformer.py:472-473), so ``if "aux_loss" in out: loss = loss + out["aux_loss"]`` - the reference
        Trainer's form - works on dense models."""
        if aux is not None:
            out["aux_loss"] = aux
        return out

    @staticmethod
    def _shift_labels(labels, labels_shifted: bool):
        if labels_shifted:
            return labels
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
        return tgt

    def loss_from_logits(self, logits, labels, labels_shifted: bool = False):
        B, S, V = logits.shape
        tgt = self._shift_labels(labels, labels_shifted)
        local = xent_ops.cross_entropy(logits.reshape(B * S, V), tgt.reshape(-1), ignore_index=-100)
        return self._loss_over_cp_group(local, tgt)

    def _loss_over_cp_group(self, local, tgt):
        if self._cp_group is None:
            return local
        # context parallel: mean over the *global* token count; gradients are summed over the CP group
        import torch.distributed as dist

        n_local = (tgt != -100).sum().float()
        n_glob = n_local.clone()
        dist.all_reduce(n_glob, group=self._cp_group)
        part = local * n_local.clamp_min(1.0) / n_glob.clamp_min(1.0)
        tot = part.detach().clone()
        dist.all_reduce(tot, group=self._cp_group)
        return part + (tot - part.detach())  # value: global mean; gradient: this rank's share

    def _collect_aux(self, ref: torch.Tensor):
        aux = None
        for blk in self.blocks.values():
            ff = getattr(blk, "feed_forward", None)
            a = getattr(ff, "aux_loss", None)
            if a is not None:
                aux = a if aux is None else aux + a
        return aux

    # ------------------------------------------------------------------ hooks
    def apply_tp(self, tp_mesh, *, fused: bool = False, sequence_parallel: bool = False, **kw):
        """Megatron TP over ``tp_mesh``. ``fused=True`` (CUDA, bf16) switches to the sequence-parallel
        layout with the all-gather fused into the column-parallel GEMMs and the reduce-scatter into the
        row-parallel ones (``ops/tp_fused.py``); activations between blocks are then row shards.
        ``sequence_parallel=True`` is the same layout through library collectives (all-gather before the
        column-parallel GEMMs, reduce-scatter behind the row-parallel ones; any device and dtype)."""
        for blk in self.blocks.values():
            blk.apply_tp(tp_mesh)
        self._tp_enabled = True
        self._tp_group = tp_mesh.get_group() if hasattr(tp_mesh, "get_group") else tp_mesh
        p0 = next(self.parameters(), None)
        on_gpu = p0 is not None and p0.is_cuda and p0.dtype == torch.bfloat16
        self._tp_host = bool(sequence_parallel and not fused) or bool(fused and not on_gpu)
        fused = bool(fused or sequence_parallel)
        self._tp_fused = fused
        self._tp_rt = None
        if fused:
            import torch.distributed as dist

            group = self._tp_group

            def reduce_hook(g):
                # the gradient of one backward pass, before it is added to ``.grad``: summing the accumulated
                # ``.grad`` instead would count earlier micro-batches once per later pass
                g = g.contiguous().clone()
                dist.all_reduce(g, group=group)
                return g

            # parameters applied to row shards (or to this rank's heads only) see a partial gradient
            for name, p in self.named_parameters():
                if "norm" in name or name.startswith("embeddings") or ".router." in name:
                    p._tp_partial = True
                    p.register_hook(reduce_hook)

            # A MoE layer is not tensor-parallel: under this layout each TP rank routes and computes its own rows, so
            # the expert (and shared-expert) weights see a partial gradient as well. Their gradients may be written by
            # kernels straight into the parameter arena, past any autograd hook, so the arena sums the regions of
            # parameters carrying ``_sp_reduce_group``; without an arena the hook below does it. The router takes its
            # load statistics over the whole TP group (``MoERouter._sp_group``).
            for m in self.modules():
                if isinstance(m, MoEBase):
                    m.mark_rows_sharded(group)

    def _ensure_tp_runtime(self, B: int, S: int, device):
        from ..models.attention import Attention
        from ..models.feed_forward import FeedForward
        from ..ops.tp_fused import HostTPRuntime, TPRuntime

        if getattr(self, "_tp_host", False):
            TPRuntime = HostTPRuntime   # noqa: N806 - same interface, library collectives
        if self._tp_rt is None or self._tp_rt.M != B * S:
            cols = self.d_model
            for m in self.modules():
                if isinstance(m, Attention):
                    cols = max(cols, (m._local_heads + 2 * m._local_kv_heads) * m.head_dim)
                elif isinstance(m, FeedForward):
                    cols = max(cols, 2 * m.w1.weight.shape[0])
            self._tp_rt = TPRuntime(self._tp_group, B * S, cols, device)
            for m in self.modules():
                if isinstance(m, (Attention, FeedForward)):
                    m._tp_rt = self._tp_rt
        self._tp_rt.batch_shape = (B, S)
        return self._tp_rt

    def apply_cp(self, cp_mesh, *, ring=None, uly=None):
        for blk in self.blocks.values():
            blk.apply_cp(cp_mesh, ring=ring, uly=uly)
        self._cp_group = cp_mesh.get_group() if hasattr(cp_mesh, "get_group") else cp_mesh
        for m in self.modules():     # a router sees 1 / cp of every sequence: its load statistics span the group
            if isinstance(m, MoEBase):
                m.router._cp_group = self._cp_group

    def replace_block_with_moe_hybrid(self, block_idx: int, moe: MoEBase, dense_ffn: Optional[FeedForward] = None):
        key = str(block_idx)
        old = self.blocks[key]
        assert isinstance(old, TransformerBlock), f"Block {block_idx} is {type(old).__name__}, not TransformerBlock"
        self.blocks[key] = MoEHybridTransformerBlock(
            d_model=self.d_model, block_idx=block_idx, n_layers=self.n_layers, attention=old.attention, moe=moe,
            dense_ffn=dense_ffn, attention_norm=old.attention_norm, moe_norm=old.feed_forward_norm,
            dropout=old.dropout.p if isinstance(old.dropout, nn.Dropout) else 0.0)

    def apply_pp(self, pp_mesh, *, num_stages: Optional[int] = None, stage_idx: Optional[int] = None,
                 split_points=None):
        """Keep only this rank's pipeline stage (blocks, plus embeddings on the first stage and the head
        on the last). With no arguments the stage is this rank's index in the PP mesh."""
        import torch.distributed as dist

        group = pp_mesh.get_group() if hasattr(pp_mesh, "get_group") else pp_mesh
        pp = dist.get_world_size(group) if group is not None else 1
        num_stages = num_stages or pp
        stage_idx = dist.get_rank(group) if stage_idx is None and group is not None else (stage_idx or 0)
        from ..parallel.pipeline_runtime import stage_layer_ranges

        lo, hi = stage_layer_ranges(self.n_layers, num_stages, split_points)[stage_idx]
        for i in range(self.n_layers):
            if not (lo <= i < hi) and str(i) in self.blocks:
                del self.blocks[str(i)]
        self._is_first_stage = stage_idx == 0
        self._is_last_stage = stage_idx == num_stages - 1
        if not self._is_first_stage and not (self.tie_word_embeddings and self._is_last_stage):
            self.embeddings = None
            self.embedding_norm = None
        if not self._is_last_stage:
            self.lm_head = None
            self.final_norm = None
        self._pp_enabled = True
        self._pp_group = group
        self._pp_stage = (stage_idx, num_stages)

    def apply_ep(self, ep_config):
        """Accepts an ``ExpertParallelConfig`` or an EP ``DeviceMesh`` / process group."""
        if not isinstance(ep_config, ExpertParallelConfig):
            import torch.distributed as dist

            group = ep_config.get_group() if hasattr(ep_config, "get_group") else ep_config
            ep_config = ExpertParallelConfig(ep_size=dist.get_world_size(group), ep_group=group)
        for blk in self.blocks.values():
            ff = getattr(blk, "feed_forward", None)
            if isinstance(ff, MoEBase):
                ff.apply_ep(ExpertParallelConfig(ep_size=ep_config.ep_size, ep_group=ep_config.ep_group,
                                                 dispatcher=ep_config.dispatcher))

    def apply_fsdp(self, dp_mesh=None, *, param_dtype=None, reduce_dtype=torch.float32, wrapping_strategy="full",
                   reshard_after_forward: bool = True, prefetch_factor: int = 0, **kw):
        from ..parallel.fsdp import MixedPrecision, shard_module

        mp = MixedPrecision(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
        for blk in self.blocks.values():
            blk.apply_fsdp(dp_mesh, wrapping_strategy=wrapping_strategy,
                           reshard_after_forward=reshard_after_forward and not self._pp_enabled, mp_policy=mp,
                           prefetch_factor=prefetch_factor)
        if self.embeddings is not None:
            shard_module(self.embeddings, dp_mesh, reshard_after_forward=reshard_after_forward, mp_policy=mp)
        if self.lm_head is not None:
            shard_module(self.lm_head, dp_mesh, reshard_after_forward=False, mp_policy=mp)
        shard_module(self, dp_mesh, reshard_after_forward=reshard_after_forward, mp_policy=mp)
        self._fsdp_enabled = True

    def apply_compile(self):
        """Kept for interface parity: the hot path is hand-written kernels, nothing is traced. Says so once, so that
        ``--compile`` is not mistaken for a speed-up."""
        if not self._compile_enabled:
            import logging

            logging.getLogger(__name__).warning(
                "apply_compile / --compile is a no-op here: the blocks already run as hand-written sm_100a kernels "
                "(and as plain PyTorch ops on CPU); nothing is traced or compiled")
        self._compile_enabled = True

    def apply_activation_checkpointing(self, mode: str = "full", block_interval: Optional[int] = None):
        from ..parallel.fsdp import apply_activation_checkpointing

        apply_activation_checkpointing(self, mode=mode, block_interval=block_interval)

    def init_weights(self, std: float = 0.02, generator: Optional[torch.Generator] = None):
        """N(0, std) for every matrix (experts use their own ``init_std``), ones for norms."""
        with torch.no_grad():
            for name, p in self.named_parameters():
                if p.dim() >= 2 and ".moe.w" not in name:
                    p.normal_(0.0, std, generator=generator)
