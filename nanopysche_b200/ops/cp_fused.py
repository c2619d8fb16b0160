"""Context-parallel attention fused into the flash kernels over peer memory.

Every rank publishes its K/V shard in symmetric memory; after one device-side barrier the attention
kernel of each rank walks the KV blocks of *all* ranks, loading the remote tiles over NVLink with
plain TMA loads from the peers' buffers (double-buffered in the kernel, so the transfer of block
``j+1`` overlaps the tensor-core work on block ``j``). There is no ring of send/recv steps and no
log-sum-exp merge between steps: one kernel sees the whole sequence. Causality is decided per
128-row block from global token positions, so the zig-zag shard layout (rank ``r`` owns chunks ``r`` and
``2cp-1-r``) gives every rank the same amount of work.

Backward: every rank publishes ``q, dO, k, v, lse, delta``; the dQ kernel pulls the peers' K/V and the
dK/dV kernel pulls the peers' Q/dO/lse/delta, so gradients never travel and need no reduction.

Replaces the reference's ring attention loop (distributed/context_parallel.py:271-330: blocking
``dist.send``/``dist.recv`` of K and V per step, dense softmax per step) and its all-to-all Ulysses
variant for the attention itself.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.distributed as dist

from . import attention as attn_ops


class CPRuntime:
    """Symmetric buffers of one context-parallel group (shared by all layers; allocated on first use)."""

    def __init__(self, group, *, zigzag: bool = True, device=None):
        self.group = group
        self.cp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.zigzag = zigzag
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.heap = None
        self._shape = None
        self._calls_f = 0
        self._calls_b = 0
        # peers are visited starting with this rank, so the ranks do not all pull from rank 0 at once
        self.order = [(self.rank + i) % self.cp for i in range(self.cp)]

    # -- layout ---------------------------------------------------------------------------------------
    def _block_positions(self, s_local: int):
        from ..parallel.context_parallel import local_positions

        assert s_local % 128 == 0 and (not self.zigzag or (s_local // 2) % 128 == 0), \
            "the fused context-parallel kernels need 128-row blocks that do not straddle zig-zag chunks"
        pos = [local_positions(s_local, self.cp, r, self.device, self.zigzag)[::128].to(torch.int32)
               for r in range(self.cp)]
        self.blk_local = pos[self.rank].contiguous()
        self.blk_all = torch.cat([pos[r] for r in self.order]).contiguous()

    def _ensure(self, q, k):
        shape = (tuple(q.shape), tuple(k.shape))
        if self._shape == shape:
            return
        assert self.heap is None, "the fused context-parallel runtime serves one (batch, sequence) shape"
        from ..parallel.symm import SymmetricHeap

        B, S, Hq, hd = q.shape
        Hkv = k.shape[2]
        qb, kb, lb = B * S * Hq * hd * 2, B * S * Hkv * hd * 2, B * Hq * S * 4
        nbytes = 2 * 2 * kb + 2 * (2 * qb + 2 * kb + 2 * lb) + (1 << 20)
        self.heap = SymmetricHeap(nbytes, self.group, self.device)
        h = self.heap
        bf, f32 = torch.bfloat16, torch.float32
        self.fwd = [dict(k=h.alloc(k.shape, bf), v=h.alloc(k.shape, bf)) for _ in range(2)]
        self.bwd = [dict(q=h.alloc(q.shape, bf), d_o=h.alloc(q.shape, bf), k=h.alloc(k.shape, bf),
                         v=h.alloc(k.shape, bf), lse=h.alloc((B, Hq, S), f32), delta=h.alloc((B, Hq, S), f32))
                    for _ in range(2)]
        self._block_positions(S)
        self._shape = shape
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _sources(self, t: torch.Tensor):
        """The buffer ``t`` on every rank in visiting order: the local tensor, raw pointers for the peers."""
        return [t if r == self.rank else self.heap.peer_ptr(t, r) for r in self.order]

    def end_step(self):
        if self.heap is not None:
            self.heap.end_step()

    # -- forward / backward ---------------------------------------------------------------------------
    def forward(self, q, k, v, causal: bool, scale: Optional[float]):
        self._ensure(q, k)
        buf = self.fwd[self._calls_f & 1]
        self._calls_f += 1
        buf["k"].copy_(k)
        buf["v"].copy_(v)
        self.heap.barrier(attn_ops.WAIT_LIMIT_NS)
        return attn_ops.flash_fwd(q, self._sources(buf["k"]), self._sources(buf["v"]), causal=causal, scale=scale,
                                  q_blk_pos=self.blk_local, k_blk_pos=self.blk_all)

    def backward(self, q, k, v, o, d_o, lse, causal: bool, scale: Optional[float]):
        buf = self.bwd[self._calls_b & 1]
        self._calls_b += 1
        buf["q"].copy_(q)
        buf["d_o"].copy_(d_o)
        buf["k"].copy_(k)
        buf["v"].copy_(v)
        buf["lse"].copy_(lse)
        attn_ops.flash_bwd(buf["q"], buf["k"], buf["v"], o, buf["d_o"], buf["lse"], causal=causal, scale=scale,
                           delta=buf["delta"], phase=1)
        self.heap.barrier(attn_ops.WAIT_LIMIT_NS)
        src = {n: self._sources(buf[n]) for n in ("k", "v", "q", "d_o", "lse", "delta")}
        dq, dk, dv, _ = attn_ops.flash_bwd(buf["q"], buf["k"], buf["v"], o, buf["d_o"], buf["lse"], causal=causal,
                                           scale=scale, delta=buf["delta"], sources=src, phase=2,
                                           q_blk_pos_local=self.blk_local, k_blk_pos_all=self.blk_all,
                                           k_blk_pos_local=self.blk_local, q_blk_pos_all=self.blk_all)
        return dq, dk, dv


class _FusedCPAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, rt: CPRuntime, causal, scale):
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        o, lse = rt.forward(q, k, v, causal, scale)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.rt, ctx.causal, ctx.scale = rt, causal, scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = ctx.rt.backward(q, k, v, o, d_o.contiguous(), lse, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None, None


def supported(q: torch.Tensor, k: torch.Tensor, cp: int, zigzag: bool) -> bool:
    s = q.shape[1]
    return (attn_ops.flash_supported(q, k) and cp <= 8 and s % 128 == 0 and (not zigzag or (s // 2) % 128 == 0)
            and q.shape[1] == k.shape[1])


def cp_attention(q, k, v, rt: CPRuntime, causal: bool = True, scale: Optional[float] = None) -> torch.Tensor:
    """Attention of the local query shard over the whole (sharded) sequence; ``[B, S/cp, H, 128]`` in and out."""
    return _FusedCPAttention.apply(q, k, v, rt, causal, scale)
