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


# ------------------------------------------------------------------------------------------ Ulysses
class UlyssesRuntime(CPRuntime):
    """Ulysses attention without the four all-to-alls: rank ``r`` computes heads ``[r H/cp, (r+1) H/cp)`` for the
    *whole* sequence by running the flash kernels once per sequence shard - Q tiles are TMA-loaded from the rank
    that owns the shard, K/V tiles from every rank, and the output rows are stored straight into the owner's
    buffer. The head/sequence exchange of the reference (distributed/context_parallel.py:334-375, four
    ``all_to_all_single`` calls) happens inside the kernels' loads and stores.

    Backward mirrors it: dQ rows are stored into the owner's buffer by the dQ kernel; dK/dV of shard ``s`` (my
    head slice) are computed by the dK/dV kernel over every rank's Q/dO and stored into rank ``s``'s buffer.
    """

    def _ensure(self, q, k):
        shape = (tuple(q.shape), tuple(k.shape))
        if self._shape == shape:
            return
        assert self.heap is None, "the fused context-parallel runtime serves one (batch, sequence) shape"
        from ..parallel.symm import SymmetricHeap

        B, S, Hq, hd = q.shape
        Hkv = k.shape[2]
        assert Hq % self.cp == 0 and Hkv % self.cp == 0, "Ulysses needs both head counts divisible by cp"
        qb, kb, lb = B * S * Hq * hd * 2, B * S * Hkv * hd * 2, B * Hq * S * 4
        nbytes = 2 * (2 * qb + 2 * kb + lb) + 2 * (3 * qb + 4 * kb + 2 * lb) + (1 << 20)
        self.heap = SymmetricHeap(nbytes, self.group, self.device)
        h = self.heap
        bf, f32 = torch.bfloat16, torch.float32
        self.fwd = [dict(q=h.alloc(q.shape, bf), k=h.alloc(k.shape, bf), v=h.alloc(k.shape, bf),
                         o=h.alloc(q.shape, bf), lse=h.alloc((B, Hq, S), f32)) for _ in range(2)]
        self.bwd = [dict(q=h.alloc(q.shape, bf), d_o=h.alloc(q.shape, bf), k=h.alloc(k.shape, bf),
                         v=h.alloc(k.shape, bf), lse=h.alloc((B, Hq, S), f32), delta=h.alloc((B, Hq, S), f32),
                         dq=h.alloc(q.shape, bf), dk=h.alloc(k.shape, bf), dv=h.alloc(k.shape, bf))
                    for _ in range(2)]
        self._block_positions(S)
        from ..parallel.context_parallel import local_positions

        self.blk_of = [local_positions(S, self.cp, r, self.device, self.zigzag)[::128].to(torch.int32).contiguous()
                       for r in range(self.cp)]
        self._shape = shape
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _head_view(self, buf: torch.Tensor, rank: int, heads_total: int):
        """``buf`` on ``rank`` restricted to this rank's head slice: (device pointer, local head count)."""
        hl = heads_total // self.cp
        return self.heap.peer_ptr(buf, rank) + self.rank * hl * buf.shape[-1] * buf.element_size(), hl

    def forward(self, q, k, v, causal, scale):
        self._ensure(q, k)
        buf = self.fwd[self._calls_f & 1]
        self._calls_f += 1
        buf["q"].copy_(q)
        buf["k"].copy_(k)
        buf["v"].copy_(v)
        self.heap.barrier(attn_ops.WAIT_LIMIT_NS)
        Hq, Hkv = q.shape[2], k.shape[2]
        ks = [self._head_view(buf["k"], r, Hkv)[0] for r in self.order]
        vs = [self._head_view(buf["v"], r, Hkv)[0] for r in self.order]
        for s in self.order:   # one launch per sequence shard: its Q rows against the whole sequence
            qp, hq = self._head_view(buf["q"], s, Hq)
            op, _ = self._head_view(buf["o"], s, Hq)
            lp = self.heap.peer_ptr(buf["lse"], s) + self.rank * hq * q.shape[1] * 4
            attn_ops.flash_fwd_raw(qp, ks, vs, op, lp, like_q=buf["q"], like_k=buf["k"], heads=(hq, Hkv // self.cp),
                                   lse_heads=Hq, causal=causal, scale=scale, q_blk_pos=self.blk_of[s],
                                   k_blk_pos=self.blk_all)
        self.heap.barrier(attn_ops.WAIT_LIMIT_NS)   # every rank's rows of my output have landed
        return buf["o"].clone(), buf["lse"].clone()

    def backward(self, q, k, v, o, d_o, lse, causal, scale):
        buf = self.bwd[self._calls_b & 1]
        self._calls_b += 1
        for name, t in (("q", q), ("d_o", d_o), ("k", k), ("v", v), ("lse", lse)):
            buf[name].copy_(t)
        attn_ops.flash_bwd(buf["q"], buf["k"], buf["v"], o, buf["d_o"], buf["lse"], causal=causal, scale=scale,
                           delta=buf["delta"], phase=1)
        self.heap.barrier(attn_ops.WAIT_LIMIT_NS)
        Hq, Hkv = q.shape[2], k.shape[2]
        hq, hkv = Hq // self.cp, Hkv // self.cp
        S = q.shape[1]
        lse_off = self.rank * hq * S * 4
        src = {n: [self._head_view(buf[n], r, Hkv if n in ("k", "v") else Hq)[0] for r in self.order]
               for n in ("k", "v", "q", "d_o")}
        src["lse"] = [self.heap.peer_ptr(buf["lse"], r) + lse_off for r in self.order]
        src["delta"] = [self.heap.peer_ptr(buf["delta"], r) + lse_off for r in self.order]
        for s in self.order:
            ptr = {n: self._head_view(buf[n], s, Hkv if n in ("k", "v", "dk", "dv") else Hq)[0]
                   for n in ("q", "d_o", "k", "v", "dq", "dk", "dv")}
            attn_ops.flash_bwd_raw(ptr, src, lse=self.heap.peer_ptr(buf["lse"], s) + lse_off,
                                   delta=self.heap.peer_ptr(buf["delta"], s) + lse_off, like_q=buf["q"],
                                   like_k=buf["k"], heads=(hq, hkv), lse_heads=Hq, causal=causal, scale=scale,
                                   blk_local=self.blk_of[s], blk_all=self.blk_all)
        self.heap.barrier(attn_ops.WAIT_LIMIT_NS)
        return buf["dq"].clone(), buf["dk"].clone(), buf["dv"].clone()


def ulysses_attention(q, k, v, rt: UlyssesRuntime, causal: bool = True, scale: Optional[float] = None):
    """Ulysses attention with the head/sequence exchange done by the kernels' loads and stores."""
    return _FusedCPAttention.apply(q, k, v, rt, causal, scale)


def ulysses_supported(q: torch.Tensor, k: torch.Tensor, cp: int, zigzag: bool) -> bool:
    return supported(q, k, cp, zigzag) and q.shape[2] % cp == 0 and k.shape[2] % cp == 0
