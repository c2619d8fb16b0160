"""Context parallelism: zig-zag sequence sharding, ring attention and Ulysses attention
(reference: distributed/context_parallel.py:50-375).

What the reference gets wrong is fixed by construction here:

* zig-zag is a real data layout: with ``cp`` ranks the sequence is cut into ``2*cp`` chunks and rank
  ``r`` owns chunks ``r`` and ``2*cp-1-r`` (equal causal work per rank). ``shard_sequence`` /
  ``unshard_sequence`` / ``local_positions`` implement it for tokens, labels and RoPE positions.
* ring steps are merged with the log-sum-exp (online softmax), fully masked pairs are skipped
  instead of producing NaN, K/V travel with their own (un-expanded) head count, and the exchange is
  a paired ``batch_isend_irecv`` on the CP group (no blocking send-then-recv deadlock).
* Ulysses re-orders the gathered sequence to natural order, so the causal mask is the ordinary one
  and attention never materialises an S x S matrix on the GPU.

The ring here is differentiable end to end (the KV rotation is an autograd function whose backward
rotates gradients the other way), which makes it the oracle for the fused sm_100a ring kernel.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import attention as attn_ops


@dataclass
class ContextParallelConfig:
    degree: int = 1
    ring: bool = True
    ulysses: bool = False
    zigzag: bool = True


# ------------------------------------------------------------------ zig-zag layout helpers
def _zigzag_order(cp: int, rank: Optional[int] = None) -> list[int]:
    """Chunk ids (of ``2*cp`` chunks) owned by ``rank``; with ``rank=None`` the global concatenation
    order of all ranks' shards."""
    if rank is not None:
        return [rank, 2 * cp - 1 - rank]
    out: list[int] = []
    for r in range(cp):
        out += [r, 2 * cp - 1 - r]
    return out


def shard_sequence(x: torch.Tensor, cp: int, rank: int, dim: int = 1, zigzag: bool = True) -> torch.Tensor:
    """This rank's shard of a full-sequence tensor (tokens, labels, hidden states)."""
    if cp <= 1:
        return x
    S = x.shape[dim]
    if zigzag:
        assert S % (2 * cp) == 0, "sequence length must be a multiple of 2*cp for zig-zag sharding"
        chunks = x.chunk(2 * cp, dim=dim)
        return torch.cat([chunks[i] for i in _zigzag_order(cp, rank)], dim=dim)
    assert S % cp == 0
    return x.chunk(cp, dim=dim)[rank]


def unshard_sequence(shards: list[torch.Tensor], cp: int, dim: int = 1, zigzag: bool = True) -> torch.Tensor:
    """Inverse of ``shard_sequence`` given every rank's shard in rank order."""
    if cp <= 1:
        return shards[0]
    if not zigzag:
        return torch.cat(shards, dim=dim)
    pieces: dict[int, torch.Tensor] = {}
    for r, s in enumerate(shards):
        a, b = s.chunk(2, dim=dim)
        pieces[r], pieces[2 * cp - 1 - r] = a, b
    return torch.cat([pieces[i] for i in range(2 * cp)], dim=dim)


def local_positions(s_local: int, cp: int, rank: int, device=None, zigzag: bool = True) -> torch.Tensor:
    """Global position of every local token ([s_local], int64)."""
    if cp <= 1:
        return torch.arange(s_local, device=device)
    if not zigzag:
        return torch.arange(s_local, device=device) + rank * s_local
    c = s_local // 2
    a, b = _zigzag_order(cp, rank)
    return torch.cat([torch.arange(c, device=device) + a * c, torch.arange(c, device=device) + b * c])


def shard_batch_for_cp(input_ids: torch.Tensor, labels: Optional[torch.Tensor], cp: int, rank: int,
                       zigzag: bool = True):
    """Shift the labels by one on the full sequence, then shard tokens and labels alike; the model is
    then called with ``labels_shifted=True``."""
    tgt = None
    if labels is not None:
        tgt = torch.full_like(labels, -100)
        tgt[:, :-1] = labels[:, 1:]
        tgt = shard_sequence(tgt, cp, rank, 1, zigzag)
    return shard_sequence(input_ids, cp, rank, 1, zigzag), tgt


def _compute_causal_mask(q_pos: torch.Tensor, k_pos: torch.Tensor) -> torch.Tensor:
    return k_pos[None, :] <= q_pos[:, None]


# ------------------------------------------------------------------ differentiable collectives
class _RingExchange(torch.autograd.Function):
    """Send ``x`` to the next rank of the ring and receive the previous rank's; backward goes the
    other way round."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _rotate(x, group, +1)

    @staticmethod
    def backward(ctx, g):
        return _rotate(g.contiguous(), ctx.group, -1), None


def _rotate(x: torch.Tensor, group, direction: int) -> torch.Tensor:
    n, r = dist.get_world_size(group), dist.get_rank(group)
    dst = dist.get_global_rank(group, (r + direction) % n)
    src = dist.get_global_rank(group, (r - direction) % n)
    x = x.contiguous()
    out = torch.empty_like(x)
    ops = [dist.P2POp(dist.isend, x, dst, group=group), dist.P2POp(dist.irecv, out, src, group=group)]
    for w in dist.batch_isend_irecv(ops):
        w.wait()
    return out


class _SeqHeadAllToAll(torch.autograd.Function):
    """[B, S/cp, H, hd] -> [B, S, H/cp, hd] (``to_heads=True``) or back; backward is the inverse."""

    @staticmethod
    def forward(ctx, x, group, to_heads):
        ctx.group, ctx.to_heads = group, to_heads
        return _a2a(x, group, to_heads)

    @staticmethod
    def backward(ctx, g):
        return _a2a(g.contiguous(), ctx.group, not ctx.to_heads), None, None


def _a2a(x: torch.Tensor, group, to_heads: bool) -> torch.Tensor:
    cp = dist.get_world_size(group)
    B, S, H, hd = x.shape
    if to_heads:  # split heads, gather sequence
        inp = x.reshape(B, S, cp, H // cp, hd).permute(2, 0, 1, 3, 4).contiguous()
        out = torch.empty_like(inp)
        dist.all_to_all_single(out, inp, group=group)
        return out.permute(1, 0, 2, 3, 4).reshape(B, cp * S, H // cp, hd)
    inp = x.reshape(B, cp, S // cp, H, hd).permute(1, 0, 2, 3, 4).contiguous()
    out = torch.empty_like(inp)
    dist.all_to_all_single(out, inp, group=group)
    return out.permute(1, 2, 0, 3, 4).reshape(B, S // cp, cp * H, hd)


def _all_to_all_single_cp2hp(x, group):
    """Sequence-sharded -> head-sharded layout (reference name)."""
    return _SeqHeadAllToAll.apply(x, group, True)


def _all_to_all_single_hp2cp(x, group):
    return _SeqHeadAllToAll.apply(x, group, False)


# ------------------------------------------------------------------ the module
_FUSED_RUNTIMES: dict = {}   # one symmetric-memory runtime per process group, shared by all layers


class RingAttention(nn.Module):
    """Context-parallel attention over ``group``: ring (default) or Ulysses.

    Inputs are this rank's sequence shard, ``q [B, S_local, Hq, hd]`` and ``k/v [B, S_local, Hkv, hd]``
    (zig-zag layout when ``use_zigzag``); the output has q's shape.
    """

    def __init__(self, group=None, use_ulysses: bool = False, use_zigzag: bool = True, *,
                 fused: Optional[bool] = None):
        super().__init__()
        self.group = group
        self.use_ulysses = use_ulysses
        self.use_zigzag = use_zigzag
        # One kernel over the peers' memory when the case allows it. ``None`` picks by measurement (B200, total sequence
        # 16384 - 32768, forward + backward): the fused ring always; fused Ulysses on 2 GPUs (3.63 ms against 3.99 ms
        # for all-to-alls around the local kernels), the all-to-all form on 4 and 8 (6.49 against 8.33 ms, 3.86
        # against 13.66 ms: every CTA of the fused form then gathers its rows from up to 7 peers one tile at a time).
        self._fused_arg = fused
        self._fused_rt = None

    @property
    def fused(self) -> bool:
        if self._fused_arg is not None:
            return bool(self._fused_arg)
        return (not self.use_ulysses) or self.cp <= 2

    @fused.setter
    def fused(self, value):
        self._fused_arg = value

    @property
    def cp(self) -> int:
        return dist.get_world_size(self.group) if self.group is not None else 1

    @property
    def rank(self) -> int:
        return dist.get_rank(self.group) if self.group is not None else 0

    def local_positions(self, s_local: int, device=None) -> torch.Tensor:
        return local_positions(s_local, self.cp, self.rank, device, self.use_zigzag)

    def global_seq_len(self, s_local: int) -> int:
        return s_local * self.cp

    def forward(self, q, k, v, cu_seqlens=None, *, causal: bool = True):
        if self.cp <= 1:
            return attn_ops.attention(q, k, v, causal=causal)
        if self.use_ulysses:
            if self.fused and q.is_cuda:
                from ..ops import cp_fused

                if cp_fused.ulysses_supported(q, k, self.cp, self.use_zigzag):
                    return cp_fused.ulysses_attention(q, k, v, self.fused_runtime(), causal=causal)
            return self._ulysses_forward(q, k, v, causal)
        if self.fused and q.is_cuda:
            from ..ops import cp_fused

            if cp_fused.supported(q, k, self.cp, self.use_zigzag):
                return cp_fused.cp_attention(q, k, v, self.fused_runtime(), causal=causal)
        return self._ring_forward(q, k, v, causal)

    def fused_runtime(self):
        """Symmetric-memory runtime of the fused kernels; one per context-parallel group."""
        if self._fused_rt is None:
            from ..ops import cp_fused

            key = (id(self.group), self.use_ulysses, self.use_zigzag)
            rt = _FUSED_RUNTIMES.get(key)
            if rt is None:
                cls = cp_fused.UlyssesRuntime if self.use_ulysses else cp_fused.CPRuntime
                rt = cls(self.group, zigzag=self.use_zigzag)
                _FUSED_RUNTIMES[key] = rt
            self._fused_rt = rt
        return self._fused_rt

    # -- ring ------------------------------------------------------------------------------------
    def _ring_forward(self, q, k, v, causal: bool):
        cp, r = self.cp, self.rank
        S = q.shape[1]
        dev = q.device
        q_pos = self.local_positions(S, dev)
        out, lse = None, None
        kv = torch.cat([k, v], dim=-1)  # one message per step
        for step in range(cp):
            src = (r - step) % cp
            k_pos = local_positions(S, cp, src, dev, self.use_zigzag)
            kk, vv = kv[..., : k.shape[-1]], kv[..., k.shape[-1]:]
            part = self._ring_step(q, kk, vv, q_pos, k_pos, causal, step, src, r)
            if part is not None:
                o_i, lse_i = part
                out, lse = (o_i, lse_i) if out is None else attn_ops.merge_attention(out, lse, o_i, lse_i)
            if step < cp - 1:
                kv = _RingExchange.apply(kv, self.group)
        return out

    def _ring_step(self, q, k, v, q_pos, k_pos, causal, step, src, r):
        """Partial attention of the local queries against the KV block of rank ``src``; with the
        zig-zag layout the visible part is a rectangle (no mask) except for the local block."""
        if not causal:
            return attn_ops.attention_ref(q, k, v, causal=False)
        if not self.use_zigzag:
            if src > r:
                return None  # the whole block is in the future
            return attn_ops.attention_ref(q, k, v, causal=True, q_pos=q_pos, k_pos=k_pos)
        c = q.shape[1] // 2
        if step == 0:
            return attn_ops.attention_ref(q, k, v, causal=True, q_pos=q_pos, k_pos=k_pos)
        if src < r:  # its first chunk precedes both of ours, its second follows both
            return attn_ops.attention_ref(q, k[:, :c], v[:, :c], causal=False)
        # src > r: only our second chunk sees the block, and sees all of it
        o2, l2 = attn_ops.attention_ref(q[:, c:], k, v, causal=False)
        o = torch.cat([torch.zeros_like(o2), o2], dim=1)
        lse = torch.cat([torch.full_like(l2, float("-inf")), l2], dim=2)
        return o, lse

    # -- Ulysses -----------------------------------------------------------------------------------
    def _ulysses_forward(self, q, k, v, causal: bool):
        cp = self.cp
        Hq, Hkv = q.shape[2], k.shape[2]
        assert Hq % cp == 0, "Ulysses needs the query head count to be a multiple of cp"
        if Hkv % cp:
            rep = cp // math.gcd(Hkv, cp)
            k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
        qh = _all_to_all_single_cp2hp(q, self.group)
        kh = _all_to_all_single_cp2hp(k, self.group)
        vh = _all_to_all_single_cp2hp(v, self.group)
        S = qh.shape[1]
        if self.use_zigzag:  # gathered order is rank-major zig-zag: put it in natural order
            c = S // (2 * cp)
            order = _zigzag_order(cp)
            perm = torch.cat([torch.arange(c, device=q.device) + order.index(i) * c for i in range(2 * cp)])
            inv = torch.empty_like(perm)
            inv[perm] = torch.arange(S, device=q.device)
            qh, kh, vh = qh[:, perm], kh[:, perm], vh[:, perm]
        o = attn_ops.attention(qh, kh, vh, causal=causal)
        if self.use_zigzag:
            o = o[:, inv]
        return _all_to_all_single_hp2cp(o.contiguous(), self.group)
