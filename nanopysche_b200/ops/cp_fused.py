"""Context-parallel attention fused into the flash kernels over peer memory.

Ring: ONE kernel per rank and pass. Its first CTAs store this rank's K|V shard into all peers' gather buffers (32 KB
chunks taken from an atomic counter) and release one arrival flag per peer; then the kernel walks the KV blocks of
*all* ranks - the local shard first, read in place - and its TMA producer waits for a source's flag the first time
it needs a tile of that source, so the remote shards arrive while the tensor cores work on what is already there. Every shard crosses NVLink once per pass (a first version
let each CTA pull its tiles straight from the peers' memory: correct, but each remote tile then crossed NVLink
once per Q block - 2.6x slower than the NCCL path, measured on 2 GPUs). There is no ring of send/recv steps and
no log-sum-exp merge between steps: one kernel sees the whole sequence. Causality is decided per 128-row block
from global token positions, so the zig-zag shard layout (rank ``r`` owns chunks ``r`` and ``2cp-1-r``) gives every
rank the same amount of work.

Backward: the shards are gathered again; the dQ kernel runs over all of them; the dK/dV kernel runs once per
source against the local Q/dO and stores its partial result into the owner's slot buffer (a reduce-scatter by peer
stores), where the ``cp`` partials are added.

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
    """Symmetric buffers of one context-parallel group (shared by all layers; allocated on first use).

    Ring attention as all-gather -> attention in one pass: every rank stores its K|V shard into all ranks' gather
    buffers (one push kernel, one arrival flag per source) and the attention kernel starts at once on the local
    blocks; its TMA producer waits for a source's flag only when it first needs a tile of that source, so the
    transfer of the remote shards overlaps the tensor-core work on what has already arrived. Each shard crosses
    NVLink once per pass. Backward: the shards are gathered again, the dQ kernel runs over all of them, and the
    dK/dV kernel runs once per source against the local Q/dO, storing its partial result straight into the owner's
    slot buffer (reduce-scatter by peer stores); the owner adds the ``cp`` partials.
    """

    def __init__(self, group, *, zigzag: bool = True, device=None):
        self.group = group
        self.cp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.zigzag = zigzag
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.heap = None
        self._shape = None
        self._calls = 0
        # sources are visited starting with this rank: its own shard needs no transfer
        self.order = [(self.rank + i) % self.cp for i in range(self.cp)]

    # -- layout ---------------------------------------------------------------------------------------
    def _block_positions(self, s_local: int):
        from ..parallel.context_parallel import local_positions

        assert s_local % 128 == 0 and (not self.zigzag or (s_local // 2) % 128 == 0), \
            "the fused context-parallel kernels need 128-row blocks that do not straddle zig-zag chunks"
        self.blk_of = [local_positions(s_local, self.cp, r, self.device, self.zigzag)[::128].to(torch.int32).contiguous()
                       for r in range(self.cp)]
        self.blk_local = self.blk_of[self.rank]
        self.blk_all = torch.cat([self.blk_of[r] for r in self.order]).contiguous()

    def _ensure(self, q, k):
        shape = (tuple(q.shape), tuple(k.shape))
        if self._shape == shape:
            return
        assert self.heap is None, "the fused context-parallel runtime serves one (batch, sequence) shape"
        from ..parallel.symm import SymmetricHeap

        kb = k.numel() * 2
        self.heap = SymmetricHeap(3 * self.cp * 2 * kb + (1 << 20), self.group, self.device)
        h = self.heap
        bf = torch.bfloat16
        self.gather = [h.alloc((self.cp, 2) + tuple(k.shape), bf) for _ in range(2)]     # [source][K|V][B,S,Hkv,hd]
        self.flags = [h.alloc((self.cp,), torch.int32) for _ in range(2)]
        self.slots = h.alloc((self.cp, 2) + tuple(k.shape), bf)                           # dK|dV partial per source
        self.ctr = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._block_positions(q.shape[1])
        self._shape = shape
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def end_step(self):
        if self.heap is not None:
            self.heap.end_step()

    def _gather_kv(self, k, v, causal):
        """Start the all-gather of this rank's K|V shard; returns the per-source K / V views (visiting order) and
        the flag descriptor the kernels wait on."""
        par = self._calls & 1
        self._calls += 1
        if causal and not self.zigzag:
            # without the zig-zag layout a rank may never touch some source, so the flags alone do not keep a
            # fast rank from overwriting a buffer a slow one still reads
            self.heap.barrier(attn_ops.WAIT_LIMIT_NS)
        h = self.heap
        e = h.next_epoch()
        # The push is part of the attention kernel: its first CTAs take 32 KB chunks of k | v from an atomic counter,
        # store them into the peers' gather buffers and the one that completes the last chunk releases this rank's
        # flag; then every CTA computes, starting with the local shard (read from k / v in place) and waiting for a
        # peer's flag only when it first needs that peer's tiles. (A separate push kernel on a second stream deadlocks
        # once the attention grid exceeds one wave: the block scheduler issues its CTAs only after all attention CTAs
        # have been issued, while the resident attention CTAs of every rank wait for each other's push.)
        self.ctr.zero_()
        nb = k.numel() * 2
        peers = self.order[1:]
        g = self.gather[par]
        push = dict(k=k, v=v, ctr=self.ctr,
                    dst=[h.peer_ptr(g, r) + self.rank * 2 * nb for r in peers],
                    flag=[h.peer_ptr(self.flags[par], r) + 4 * self.rank for r in peers])
        flags = dict(flags=self.flags[par], idx=[-1] + peers, epoch=e, epoch_base=h.epoch_base, which=1, push=push)
        return [k] + [g[r, 0] for r in peers], [v] + [g[r, 1] for r in peers], flags

    # -- forward / backward ---------------------------------------------------------------------------
    def forward(self, q, k, v, causal: bool, scale: Optional[float]):
        self._ensure(q, k)
        ks, vs, flags = self._gather_kv(k, v, causal)
        res = attn_ops.flash_fwd(q, ks, vs, causal=causal, scale=scale, q_blk_pos=self.blk_local,
                                 k_blk_pos=self.blk_all, flags=flags)
        return res

    def backward(self, q, k, v, o, d_o, lse, causal: bool, scale: Optional[float]):
        ks, vs, flags = self._gather_kv(k, v, causal)
        # delta + dQ over every source's K/V (waits for the shards as they arrive)
        dq, _, _, delta = attn_ops.flash_bwd(q, k, v, o, d_o, lse, causal=causal, scale=scale, phase=3, skip=2,
                                             sources=dict(k=ks, v=vs), flags=flags,
                                             q_blk_pos_local=self.blk_local, k_blk_pos_all=self.blk_all)
        # dK/dV of every source's shard against the local Q/dO, stored into the owner's slot for this rank
        for i, r in enumerate(self.order):
            dst = self.heap.peer_ptr(self.slots[self.rank], r)
            half = k.numel() * 2
            attn_ops.flash_bwd(q, ks[i], vs[i], o, d_o, lse, causal=causal, scale=scale, delta=delta, phase=2, skip=1,
                               out=(None, dst, dst + half),
                               k_blk_pos_local=self.blk_of[r], q_blk_pos_all=self.blk_local)
        self.heap.barrier(attn_ops.WAIT_LIMIT_NS)   # every rank's partials for my shard have landed
        red = self.slots.float().sum(0)
        return dq, red[0].to(torch.bfloat16), red[1].to(torch.bfloat16)


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
    """Ulysses attention with the all-to-alls inside push kernels and the attention kernels' stores.

    Rank ``r`` computes heads ``[r H/cp, (r+1) H/cp)`` for the whole sequence. One push kernel per tensor stores
    head slice ``p`` of this rank's q / k / v shard into rank ``p``'s gather buffers (every element crosses NVLink
    once) and releases one arrival flag; the flash kernels then run once per sequence shard on local memory,
    waiting for a shard's flag when they first touch it, and store their output rows straight into the buffer of
    the rank that owns the shard. The four ``all_to_all_single`` calls of the reference
    (distributed/context_parallel.py:334-375) become two push kernels overlapped with the attention and the
    kernels' own epilogue stores. Backward mirrors it with q, dO, k, v, lse and delta pushed and dQ / dK / dV
    stored to their owners.
    """

    def _ensure(self, q, k):
        shape = (tuple(q.shape), tuple(k.shape))
        if self._shape == shape:
            return
        assert self.heap is None, "the fused context-parallel runtime serves one (batch, sequence) shape"
        from ..parallel.symm import SymmetricHeap

        B, S, Hq, hd = q.shape
        Hkv = k.shape[2]
        cp = self.cp
        assert Hq % cp == 0 and Hkv % cp == 0, "Ulysses needs both head counts divisible by cp"
        self.hq, self.hkv = Hq // cp, Hkv // cp
        qb, kb, lb = q.numel() * 2, k.numel() * 2, B * Hq * S * 4
        self.heap = SymmetricHeap(2 * (2 * qb + 2 * kb + 2 * lb) + 2 * qb + 2 * kb + lb + (1 << 20), self.group,
                                  self.device)
        h = self.heap
        bf, f32 = torch.bfloat16, torch.float32
        gq, gk, gl = (cp, B, S, self.hq, hd), (cp, B, S, self.hkv, hd), (cp, B, self.hq, S)
        # gather buffers [source rank][...my head slice...], double-buffered by call parity
        self.g = [dict(q=h.alloc(gq, bf), d_o=h.alloc(gq, bf), k=h.alloc(gk, bf), v=h.alloc(gk, bf),
                       lse=h.alloc(gl, f32), delta=h.alloc(gl, f32)) for _ in range(2)]
        self.flags = [h.alloc((cp,), torch.int32) for _ in range(2)]
        # results written by the peers: every rank stores its head slice of my rows
        self.res = dict(o=h.alloc(q.shape, bf), lse=h.alloc((B, Hq, S), f32), dq=h.alloc(q.shape, bf),
                        dk=h.alloc(k.shape, bf), dv=h.alloc(k.shape, bf))
        self.ctr = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._block_positions(S)
        self._shape = shape
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _push(self, par: int, items, epoch: int):
        """All-to-all by peer stores of ``items`` = [(name, tensor [rows..., H, ...])]; the last one sets the flag."""
        import ctypes as C

        from . import _lib

        h = self.heap
        for i, (name, t) in enumerate(items):
            t = t if t.is_contiguous() else t.contiguous()
            if name in ("lse", "delta"):
                rows, row_bytes = t.shape[0], t.shape[1] * t.shape[2] * 4           # [B, Hq, S]: rows = batch
            else:
                rows, row_bytes = t.shape[0] * t.shape[1], t.shape[2] * t.shape[3] * 2   # [B, S, H, hd]: rows = tokens
            last = i == len(items) - 1
            _lib.check(_lib.lib().np_a2a_push(
                C.c_void_p(t.data_ptr()), C.c_longlong(rows), C.c_longlong(row_bytes),
                h.host_ptr_array(self.g[par][name]), h.host_ptr_array(self.flags[par]), C.c_void_p(self.ctr.data_ptr()),
                self.rank, self.cp, epoch, C.c_void_p(h.epoch_base.data_ptr()), int(last), 64,
                C.c_void_p(_lib.stream())), "a2a_push")

    def _head_ptr(self, buf: torch.Tensor, rank: int, heads_total: int) -> int:
        """Address of this rank's head slice inside ``buf`` ([B, S, H, hd]) on ``rank``."""
        return self.heap.peer_ptr(buf, rank) + self.rank * (heads_total // self.cp) * buf.shape[-1] * 2

    def forward(self, q, k, v, causal, scale):
        self._ensure(q, k)
        par = self._calls & 1
        self._calls += 1
        h = self.heap
        e = h.next_epoch()
        self._push(par, [("q", q), ("k", k), ("v", v)], e)
        g = self.g[par]
        Hq, S = q.shape[2], q.shape[1]
        ks, vs = [g["k"][r] for r in self.order], [g["v"][r] for r in self.order]
        for s in self.order:   # one launch per sequence shard: its Q rows against the whole sequence
            flags = dict(flags=self.flags[par], idx=self.order, epoch=e, epoch_base=h.epoch_base, own=s)
            attn_ops.flash_fwd_raw(g["q"][s].data_ptr(), ks, vs, self._head_ptr(self.res["o"], s, Hq),
                                   h.peer_ptr(self.res["lse"], s) + self.rank * self.hq * S * 4,
                                   like_q=g["q"][s], like_k=g["k"][s], like_o=q, heads=(self.hq, self.hkv), lse_heads=Hq,
                                   causal=causal, scale=scale, q_blk_pos=self.blk_of[s], k_blk_pos=self.blk_all,
                                   flags=flags)
        h.barrier(attn_ops.WAIT_LIMIT_NS)   # every rank's slice of my output rows has landed
        return self.res["o"].clone(), self.res["lse"].clone()

    def backward(self, q, k, v, o, d_o, lse, causal, scale):
        par = self._calls & 1
        self._calls += 1
        h = self.heap
        _, _, _, delta = attn_ops.flash_bwd(q, k, v, o, d_o, lse, causal=causal, scale=scale, phase=1)
        e = h.next_epoch()
        self._push(par, [("q", q), ("d_o", d_o), ("k", k), ("v", v), ("lse", lse), ("delta", delta)], e)
        g = self.g[par]
        Hq, Hkv = q.shape[2], k.shape[2]
        src = {n: [g[n][r] for r in self.order] for n in ("k", "v", "q", "d_o", "lse", "delta")}
        for s in self.order:
            ptr = dict(q=g["q"][s].data_ptr(), d_o=g["d_o"][s].data_ptr(), k=g["k"][s].data_ptr(), v=g["v"][s].data_ptr(),
                       dq=self._head_ptr(self.res["dq"], s, Hq), dk=self._head_ptr(self.res["dk"], s, Hkv),
                       dv=self._head_ptr(self.res["dv"], s, Hkv))
            flags = dict(flags=self.flags[par], idx=self.order, epoch=e, epoch_base=h.epoch_base, own=s, which=3)
            attn_ops.flash_bwd_raw(ptr, src, lse=g["lse"][s].data_ptr(), delta=g["delta"][s].data_ptr(),
                                   like_q=g["q"][s], like_k=g["k"][s], like_dq=q, like_dk=k, heads=(self.hq, self.hkv),
                                   lse_heads=self.hq, causal=causal, scale=scale, blk_local=self.blk_of[s],
                                   blk_all=self.blk_all, flags=flags)
        h.barrier(attn_ops.WAIT_LIMIT_NS)
        return self.res["dq"].clone(), self.res["dk"].clone(), self.res["dv"].clone()


def ulysses_attention(q, k, v, rt: UlyssesRuntime, causal: bool = True, scale: Optional[float] = None):
    """Ulysses attention with the head/sequence exchange done by the kernels' loads and stores."""
    return _FusedCPAttention.apply(q, k, v, rt, causal, scale)


def ulysses_supported(q: torch.Tensor, k: torch.Tensor, cp: int, zigzag: bool) -> bool:
    return supported(q, k, cp, zigzag) and q.shape[2] % cp == 0 and k.shape[2] % cp == 0
