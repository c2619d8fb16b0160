"""Fully-sharded (ZeRO-3 style) linear layers with the collectives inside the GEMMs.

Each rank owns ``N/n`` rows of a weight ``[N, K]``.

* forward   : every rank stores its row shard into all ranks' gather buffers (one push kernel) and the tcgen05
              GEMM ``y = x W^T`` starts right away: its TMA producer waits for the arrival flag of the shard a
              tile's B rows belong to, so tiles of shards that have landed run while later shards are still
              on the wire (parameter all-gather fused into the first consuming GEMM).
* dgrad     : the shards are gathered again (the buffer is shared by all layers) and ``dx = dy W`` waits per
              K-slice of B in the same way.
* wgrad     : ``dW = dy^T x`` is computed for all ``N`` rows into this rank's symmetric buffer; after a device
              barrier every rank sums its row shard over all ranks' buffers with peer loads (reduce-scatter).

Replaces ``fully_shard`` (reference: distributed/fsdp.py:18-83: NCCL all-gather before every layer forward and
backward, NCCL reduce-scatter after backward).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from .attention import WAIT_LIMIT_NS
from .gemm import gemm


class FSDPRuntime:
    """Gather / slot buffers and flag tables for one shard group, shared by every sharded linear."""

    def __init__(self, group, max_weight_elems: int, device=None):
        from ..parallel.symm import SymmetricHeap

        self.group = group
        self.n = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.max_elems = max_weight_elems
        self.heap = SymmetricHeap(4 * max_weight_elems * 2 + (1 << 20), group, self.device)
        h = self.heap
        self.gather = [h.alloc((max_weight_elems,), torch.bfloat16) for _ in range(2)]
        self.slots = h.alloc((max_weight_elems,), torch.bfloat16)
        self.partial = [self.slots, h.alloc((max_weight_elems,), torch.bfloat16)]   # wgrad partials, by call parity
        self._rs_calls = 0
        self.ag_flags = [h.alloc((self.n,), torch.int32) for _ in range(2)]
        self.rs_flags = h.alloc((self.n,), torch.int32)
        self.p_slots = h.ptr_array(self.slots)
        self.p_done_flag = torch.tensor([h.peer_ptr(self.rs_flags, s) + 4 * self.rank for s in range(self.n)],
                                        dtype=torch.int64, device=self.device)
        self.done_counters = torch.zeros(self.n, dtype=torch.int32, device=self.device)
        self.ctr = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.sent = torch.ones(self.n, dtype=torch.int32, device=self.device)
        self._calls = 0
        self._tables: dict = {}

        torch.cuda.synchronize()
        dist.barrier(group=group)

    def end_step(self):
        self.heap.end_step()

    @staticmethod
    def supported(n_rows: int, world: int) -> bool:
        return n_rows % world == 0 and (n_rows // world) % 128 == 0

    def _rs_tables(self, N: int):
        t = self._tables.get(N)
        if t is None:
            ns = N // self.n
            r = torch.arange(N, device=self.device)
            owner, local = r // ns, r % ns
            t = dict(row_dst=(owner << 40) | (local * self.n + self.rank),
                     mblk_owner=((torch.arange(N // 128, device=self.device) * 128) // ns).to(torch.int32),
                     done_expected=torch.full((self.n,), ns // 128, dtype=torch.int32, device=self.device),
                     slot_pos=torch.zeros((ns, self.n), dtype=torch.int32, device=self.device))
            self._tables[N] = t
        return t

    # -- building blocks ---------------------------------------------------------------------------------
    def gather_push(self, w_shard: torch.Tensor):
        """Start the all-gather of a row-sharded weight; returns (full view [N, K], flags tensor, epoch)."""
        ns, K = w_shard.shape
        assert ns * self.n * K <= self.max_elems and w_shard.is_contiguous() and w_shard.dtype == torch.bfloat16
        par = self._calls & 1
        self._calls += 1
        e = self.heap.next_epoch()
        h = self.heap
        _lib.check(_lib.lib().np_allgather_push(
            C.c_void_p(w_shard.data_ptr()), h.host_ptr_array(self.gather[par]), C.c_longlong(ns * K * 2),
            h.host_ptr_array(self.ag_flags[par]), C.c_void_p(self.ctr.data_ptr()), self.rank, self.n, e,
            C.c_void_p(h.epoch_base.data_ptr()), 0, C.c_void_p(_lib.stream())), "fsdp_gather_push")
        return self.gather[par][: ns * self.n * K].view(ns * self.n, K), self.ag_flags[par], e

    def ag_gemm(self, A: torch.Tensor, w_shard: torch.Tensor):
        """``A @ all_gather(w_shard)^T`` as ONE kernel (shard rows a multiple of 256): the GEMM's CTAs first store
        their slice of the shard into every rank's gather buffer and release this rank's flag, then compute the
        output columns of the own shard (read in place) and a peer's columns once its flag has arrived."""
        ns, K = w_shard.shape
        assert ns % 256 == 0 and ns * self.n * K <= self.max_elems and w_shard.is_contiguous()
        par = self._calls & 1
        self._calls += 1
        h = self.heap
        e = h.next_epoch()
        N = ns * self.n
        full = self.gather[par][: N * K].view(N, K)
        out = torch.empty((A.shape[0], N), device=A.device, dtype=torch.bfloat16)
        nbytes = ns * K * 2
        dst = (C.c_void_p * self.n)(*[h.peer_ptr(self.gather[par], r) + self.rank * nbytes for r in range(self.n)])
        flg = (C.c_void_p * self.n)(*[h.peer_ptr(self.ag_flags[par], r) + 4 * self.rank for r in range(self.n)])
        g = _lib.GemmArgs()
        g.A, g.B, g.C = A.data_ptr(), full.data_ptr(), out.data_ptr()
        g.lda, g.ldb, g.ldc = A.stride(0), K, N
        g.a_rows, g.b_rows = A.shape[0], N
        g.M, g.N, g.K = A.shape[0], N, K
        g.mode, g.alpha, g.bn = 0, 1.0, 256
        g.b_ready_flags, g.b_rows_per_flag = self.ag_flags[par].data_ptr(), ns
        g.B_loc, g.ldb_loc = w_shard.data_ptr(), K
        g.b_loc_lo, g.b_loc_hi = self.rank * ns, (self.rank + 1) * ns
        g.b_local_flag = self.rank + 1
        g.n_rot = self.rank * ns // 256
        g.push_src, g.push_bytes, g.push_n = w_shard.data_ptr(), nbytes, self.n
        g.push_dst, g.push_flag = C.cast(dst, C.c_void_p), C.cast(flg, C.c_void_p)
        g.push_ctr = self.ctr.data_ptr()
        g.epoch, g.flag_limit_ns = e, WAIT_LIMIT_NS
        g.epoch_base = h.epoch_base.data_ptr()
        _lib.check(_lib.lib().np_gemm_bf16(C.byref(g), C.c_void_p(_lib.stream())), "fsdp_ag_gemm")
        return out

    def gemm_b_arriving(self, A, W_full, flags, epoch, rows_per_flag, *, b_mn: bool, w_local=None):
        """``A @ W^T`` (``b_mn=False``) or ``A @ W`` (``b_mn=True``) while W's row shards are still arriving. With
        ``w_local`` (this rank's shard, forward layout only) the own rows are read from it without a flag and their
        tiles come first."""
        M, K = A.shape
        N = W_full.shape[1] if b_mn else W_full.shape[0]
        out = torch.empty((M, N), device=A.device, dtype=torch.bfloat16)
        g = _lib.GemmArgs()
        g.A, g.B, g.C = A.data_ptr(), W_full.data_ptr(), out.data_ptr()
        g.lda, g.ldb, g.ldc = A.stride(0), W_full.stride(0), N
        g.a_rows, g.b_rows = A.shape[0], W_full.shape[0]
        g.M, g.N, g.K = M, N, K
        g.b_mn, g.mode, g.alpha = int(b_mn), 0, 1.0
        g.b_ready_flags, g.b_rows_per_flag = flags.data_ptr(), rows_per_flag
        if w_local is not None and not b_mn and rows_per_flag % 256 == 0:
            g.B_loc, g.ldb_loc = w_local.data_ptr(), w_local.stride(0)
            g.b_loc_lo, g.b_loc_hi = self.rank * rows_per_flag, (self.rank + 1) * rows_per_flag
            g.b_local_flag = self.rank + 1
            g.bn = 256
            g.n_rot = self.rank * rows_per_flag // 256
        g.epoch, g.flag_limit_ns = epoch, WAIT_LIMIT_NS
        g.epoch_base = self.heap.epoch_base.data_ptr()
        _lib.check(_lib.lib().np_gemm_bf16(C.byref(g), C.c_void_p(_lib.stream())), "fsdp_gemm")
        return out

    def wgrad_reduce_scatter(self, dy, x):
        """``reduce_scatter(dy^T x)`` over the weight rows: this rank's ``[N/n, K]`` gradient shard. The wgrad GEMM
        writes the full partial ``[N, K]`` into this rank's symmetric buffer; after a device barrier every rank sums
        its row shard over all ranks' buffers with peer loads."""
        T, N = dy.shape
        K = x.shape[1]
        assert N * K <= self.max_elems
        buf = self.partial[self._rs_calls & 1]
        self._rs_calls += 1
        part = buf[: N * K].view(N, K)
        gemm(dy, x, a_mn=True, b_mn=True, out=part)
        self.heap.barrier(WAIT_LIMIT_NS)
        ns = N // self.n
        out = torch.empty((ns, K), device=dy.device, dtype=torch.bfloat16)
        _lib.check(_lib.lib().np_rs_reduce_bf16(
            self.heap.host_ptr_array(buf), self.n, C.c_longlong(self.rank * ns * K), C.c_longlong(ns * K),
            C.c_void_p(out.data_ptr()), C.c_void_p(_lib.stream())), "fsdp_rs_reduce")
        return out


class _ShardedLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_shard, rt: FSDPRuntime):
        x2 = x.reshape(-1, x.shape[-1])
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        if w_shard.shape[0] % 256 == 0:
            y = rt.ag_gemm(x2, w_shard)           # push + GEMM in one kernel
        else:
            full, flags, e = rt.gather_push(w_shard)
            y = rt.gemm_b_arriving(x2, full, flags, e, w_shard.shape[0], b_mn=False, w_local=w_shard)
        ctx.save_for_backward(x2, w_shard)
        ctx.rt, ctx.x_shape = rt, x.shape
        return y.view(*x.shape[:-1], y.shape[-1])

    @staticmethod
    def backward(ctx, dy):
        x2, w_shard = ctx.saved_tensors
        rt = ctx.rt
        dy2 = dy.reshape(-1, dy.shape[-1])
        dy2 = dy2 if dy2.is_contiguous() else dy2.contiguous()
        full, flags, e = rt.gather_push(w_shard)   # the parameters are gathered again, not kept
        dx = rt.gemm_b_arriving(dy2, full, flags, e, w_shard.shape[0], b_mn=True)
        dw = rt.wgrad_reduce_scatter(dy2, x2)
        return dx.view(ctx.x_shape), dw.to(w_shard.dtype), None


def sharded_linear(x: torch.Tensor, w_shard: torch.Tensor, rt: FSDPRuntime) -> torch.Tensor:
    """``x @ all_gather(w_shard)^T`` with the all-gather inside the GEMM; gradients arrive reduce-scattered."""
    return _ShardedLinear.apply(x, w_shard, rt)
