"""Fused MoE layer on sm_100a: router -> capacity -> dispatch (peer stores) -> grouped SwiGLU GEMM
(waits on arrival flags) -> grouped down GEMM (epilogue pushes rows back to their source rank and
signals it) -> combine, with the mirrored backward. One autograd node per layer; nothing in it
synchronises with the host, and with one rank the "peers" are this GPU itself, so the same kernels
run at every EP degree.

Replaces, in the reference: the router (model/moe.py:133-321), the capacity loop (:1395-1448), the
NCCL dispatcher with its 4 collectives and 3 host syncs per layer (:360-498), the per-expert Python
loop of matmuls (:1498-1596) and the scatter-back (:1386-1390).

Buffer protocol (all in the symmetric heap, same offsets on every rank):
  recv_x[layer]  rows pushed by the sources, region ``[local expert][source rank]`` of ``R`` rows
  ret_y[layer]   expert outputs returned to the source, one row per (token, k) slot
  recv_g, ret_g  the same two roles for the backward pass (shared by all layers)
  mblk_rows, row_dst, src_blocks   per-block row counts / per-row return addresses / block counts,
                 written by the sources together with the rows
  dispatch_flags[src], combine_flags[peer]   monotone epochs: "rows of epoch e have landed"
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

from . import _lib
from .activation import glu, glu_bwd

GATING_IDS = {"softmax": 0, "sigmoid": 1}
WAIT_LIMIT_NS = int(os.environ.get("NPB200_WAIT_LIMIT_MS", "10000")) * 1_000_000


# ------------------------------------------------------------------------------------------------ router
class _Router(torch.autograd.Function):
    """logits -> top-k -> gating weights, with the load-balance / z-loss statistics in the same pass."""

    @staticmethod
    def forward(ctx, x2, gate_w, gate_b, score_bias, K, gating, coef_z):
        T, D = x2.shape
        E = gate_w.shape[0]
        dev = x2.device
        logits = torch.empty((T, E), device=dev, dtype=torch.float32)
        _lib.call("router_logits", x2, gate_w, gate_b, logits, T, D, E)
        weights = torch.empty((T, K), device=dev, dtype=torch.float32)
        indices = torch.empty((T, K), device=dev, dtype=torch.int32)
        stats = torch.zeros(2 * E + 1, device=dev, dtype=torch.float32)
        counts = torch.zeros(E, device=dev, dtype=torch.int32)
        _lib.call("router_topk", logits, score_bias, weights, indices, counts, stats[:E], stats[E:E + 1], T, E, K,
                  gating)
        f = counts.float() / T
        aux = E * (f * (stats[:E] / T)).sum()
        if coef_z:
            aux = aux + coef_z * stats[E] / T
        ctx.save_for_backward(x2, gate_w, logits, weights, indices, f, score_bias if score_bias is not None
                              else logits.new_empty(0))
        ctx.cfg = (K, gating, float(coef_z or 0.0), score_bias is not None)
        ctx.mark_non_differentiable(indices, counts)
        return weights, indices, aux, counts

    @staticmethod
    def backward(ctx, dweights, _di, daux, _dc):
        x2, gate_w, logits, weights, indices, f, sb = ctx.saved_tensors
        K, gating, coef_z, has_sb = ctx.cfg
        T, E = logits.shape
        D = x2.shape[1]
        dl = torch.empty_like(logits)
        dw = dweights.contiguous() if dweights is not None else None
        da = daux.reshape(1).float().contiguous() if daux is not None else None
        _lib.call("router_bwd", logits, sb if has_sb else None, weights, indices, dw, f, da, 1.0, coef_z, dl, T, E, K,
                  gating)
        parts = _lib.lib().np_router_dgate_parts(T)
        scratch = torch.empty((parts, E, D), device=x2.device, dtype=torch.float32)
        dgw = torch.empty_like(gate_w)
        dgb = torch.empty(E, device=x2.device, dtype=torch.float32)
        _lib.call("router_dgate", dl, x2, dgw, dgb, scratch, T, D, E, 0)
        if x2.dtype == torch.bfloat16 and gate_w.dtype == torch.float32 and gate_w.is_contiguous():
            dx = torch.empty_like(x2)
            _lib.call("router_dx", dl, gate_w, dx, T, D, E)
        else:
            dx = (dl @ gate_w.float()).to(x2.dtype)
        return dx, dgw, dgb, None, None, None, None


def route(x: torch.Tensor, router) -> tuple:
    """Kernel path of ``MoERouter.forward`` for bf16 CUDA input: (weights, indices int64, aux, counts)."""
    cfg = router.config
    D = x.shape[-1]
    x2 = x.reshape(-1, D)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    gating = GATING_IDS[getattr(cfg.gating_function, "value", cfg.gating_function)]
    w, idx, aux, counts = _Router.apply(x2, router.gate.weight, router.gate.bias, router.score_bias, router.top_k,
                                        gating, cfg.z_loss_multiplier or 0.0)
    lead = x.shape[:-1]
    return w.view(*lead, -1), idx.long().view(*lead, -1), aux, counts


# ------------------------------------------------------------------------------------------------ runtime
class FusedMoERuntime:
    """Symmetric buffers, flags and static tables shared by all MoE layers of one model replica."""

    def __init__(self, *, tokens: int, d_model: int, hidden: int, num_experts: int, top_k: int, n_layers: int,
                 capacity_factor: Optional[float], group=None, device=None, max_ctas_dispatch: int = 0,
                 fp8: bool = False):
        import torch.distributed as dist

        from ..parallel.symm import SymmetricHeap

        self.group = group
        self.N = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.N > 1 else 0
        self.T, self.D, self.H, self.E, self.K, self.L = tokens, d_model, hidden, num_experts, top_k, n_layers
        assert num_experts % self.N == 0
        self.E_local = num_experts // self.N
        self.capacity = int(capacity_factor * tokens / num_experts) if capacity_factor is not None else -1
        cap_rows = min(self.capacity, tokens) if self.capacity >= 0 else tokens
        self.R = max(128, (cap_rows + 127) // 128 * 128)
        self.bpr = self.R // 128
        self.rows_total = self.E_local * self.N * self.R
        self.blocks = self.rows_total // 128
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        row_bytes = self.rows_total * d_model * 2
        slot_bytes = tokens * top_k * d_model * 2
        self.fp8 = bool(fp8) and d_model % 256 == 0 and hidden % 128 == 0   # 128-wide scale blocks on both GEMMs
        need = n_layers * (row_bytes + slot_bytes) + row_bytes + slot_bytes + self.rows_total * 8 + (1 << 20)
        if self.fp8:  # e4m3 rows + their exponent chunks (512 bytes per 128 rows x 128 columns) per layer
            need += n_layers * (self.rows_total * d_model + self.rows_total * (d_model // 128) * 4 + 8192)
        self.heap = SymmetricHeap(need, group, self.device)
        h = self.heap
        self.recv_x = [h.alloc((self.rows_total, d_model), torch.bfloat16) for _ in range(n_layers)]
        self.ret_y = [h.alloc((tokens * top_k, d_model), torch.bfloat16) for _ in range(n_layers)]
        self.recv_xq = self.recv_xs = self.p_recv_xq = self.p_recv_xs = None
        if self.fp8:
            self.recv_xq = [h.alloc((self.rows_total, d_model), torch.uint8) for _ in range(n_layers)]
            # exponent bytes of the 1x128 blocks in the chunk layout of the block-scaled MMA: 4 bytes per row and block
            self.recv_xs = [h.alloc((self.rows_total * (d_model // 128) * 4,), torch.uint8) for _ in range(n_layers)]
            self.p_recv_xq = [h.ptr_array(t) for t in self.recv_xq]
            self.p_recv_xs = [h.ptr_array(t) for t in self.recv_xs]
        self.recv_g = h.alloc((self.rows_total, d_model), torch.bfloat16)
        self.ret_g = h.alloc((tokens * top_k, d_model), torch.bfloat16)
        self.row_dst = h.alloc((self.rows_total,), torch.int64)
        self.mblk_rows = h.alloc((self.blocks,), torch.int32)
        self.src_blocks = h.alloc((self.N,), torch.int32)
        self.dispatch_flags = h.alloc((self.N,), torch.int32)
        self.combine_flags = h.alloc((self.N,), torch.int32)
        # peer pointer tables
        self.p_recv_x = [h.ptr_array(t) for t in self.recv_x]
        self.p_ret_y = [h.ptr_array(t) for t in self.ret_y]
        self.p_recv_g, self.p_ret_g = h.ptr_array(self.recv_g), h.ptr_array(self.ret_g)
        self.p_row_dst, self.p_mblk_rows = h.ptr_array(self.row_dst), h.ptr_array(self.mblk_rows)
        self.p_src_blocks = h.ptr_array(self.src_blocks)
        self.p_dispatch_flags = h.ptr_array(self.dispatch_flags)
        # the flag a peer releases when all rows destined to rank s are stored: combine_flags[self.rank] on s
        self.p_done_flag = torch.tensor([h.peer_ptr(self.combine_flags, s) + 4 * self.rank for s in range(self.N)],
                                        dtype=torch.int64, device=self.device)
        # static per-block tables: group (local expert) and flag index (source rank)
        blk = torch.arange(self.blocks, device=self.device)
        self.mblk_group = (blk // (self.N * self.bpr)).to(torch.int32)
        self.mblk_flag = ((blk // self.bpr) % self.N).to(torch.int32)
        self.done_counters = torch.zeros(self.N, device=self.device, dtype=torch.int32)
        self.dispatch_ctr = torch.zeros(1, device=self.device, dtype=torch.int32)
        self.layer_of: dict[int, int] = {}
        self.max_ctas_dispatch = max_ctas_dispatch
        self._wq: dict[int, tuple] = {}        # per layer: quantised expert weights (buffers reused every step)
        self._wq_valid: set[int] = set()       # layers whose quantised weights match the current bf16 weights
        # DeepSeek-V3 auxiliary-loss-free balancing, kept on the device: per-layer assignment counts of the step and
        # one [layers, experts] tensor that every router's ``score_bias`` is a row of (``bind_router_bias``)
        h.reserve_allreduce(max(64, n_layers * num_experts))
        self.bias_counts = torch.zeros((n_layers, num_experts), device=self.device, dtype=torch.float32)
        self.score_bias_all: Optional[torch.Tensor] = None
        self.extra_count_groups: list = []   # process groups whose ranks' load counts join the bias update
        self.bias_coef = 0.0
        if self.N > 1:
            torch.cuda.synchronize()
            dist.barrier(group=group)

    def layer_index(self, module) -> int:
        k = id(module)
        if k not in self.layer_of:
            self.layer_of[k] = len(self.layer_of)
            assert self.layer_of[k] < self.L, "more MoE layers than the runtime was sized for"
        return self.layer_of[k]

    def next_epoch(self) -> int:
        return self.heap.next_epoch()

    def bind_router_bias(self, moe_modules):
        """Make the routers' ``score_bias`` buffers rows of one tensor so that the per-step update of all layers
        (reference: model/moe.py:293-321, there a host-side loop with two world all-reduces per layer that nothing
        calls) is a handful of small launches with no host synchronisation, capturable in the step's graph."""
        cfg = moe_modules[0].router.config
        self.score_bias_all = torch.zeros((self.L, self.E), device=self.device, dtype=torch.float32)
        self.bias_coef = float(cfg.bias_update_sign) * float(cfg.bias_gamma)
        for m in moe_modules:
            row = self.score_bias_all[self.layer_index(m)]
            row.copy_(m.router.score_bias)
            m.router.score_bias = row
            m.router._device_side_update = True

    def update_router_bias(self):
        """``bias += sign * gamma * (load fraction - 1/E)`` for every layer from this step's counts, summed over the
        expert-parallel ranks through peer memory. Runs once per optimizer step, before ``end_step``."""
        if self.score_bias_all is None:
            return
        c = self.bias_counts
        if self.N > 1:
            self.heap.all_reduce_(c.view(-1))
        # other ranks that hold the same layers and route other tokens (data-parallel copies of the expert shards,
        # context-parallel peers, TP peers under sequence parallelism): set by engine.prepare_training, empty for
        # expert parallelism over all ranks, where the step stays free of library collectives
        if self.extra_count_groups:
            import torch.distributed as dist

            for g in self.extra_count_groups:
                dist.all_reduce(c, group=g)
        tot = c.sum(dim=1, keepdim=True).clamp_min_(1.0)
        self.score_bias_all.add_((c / tot).sub_(1.0 / self.E), alpha=self.bias_coef)
        c.zero_()

    def end_step(self):
        self.heap.end_step()
        self._wq_valid.clear()   # the optimizer has written new weights

    def quantised_weights(self, layer: int, w1, w3, w2):
        """e4m3 copies of a layer's expert weights with 128x128 power-of-two block scales, made once per optimizer
        step (every forward of a gradient-accumulation step reuses them): ``[gate; up]`` stacked per expert for a
        single gate|up GEMM, and the down projection transposed per expert to ``[D, H]``."""
        from .gemm_mxfp8 import flow_quantize_weight, sf_bytes

        E_l, H, D = self.E_local, self.H, self.D
        if layer not in self._wq:
            dev = self.device
            self._wq[layer] = (torch.empty((E_l * 2 * H, D), device=dev, dtype=torch.float8_e4m3fn),
                               torch.empty((sf_bytes(E_l * 2 * H, D),), device=dev, dtype=torch.uint8),
                               torch.empty((E_l * D, H), device=dev, dtype=torch.float8_e4m3fn),
                               torch.empty((sf_bytes(E_l * D, H),), device=dev, dtype=torch.uint8))
        w13q, s13, w2q, s2 = self._wq[layer]
        if layer not in self._wq_valid:
            flow_quantize_weight(w1.detach(), E_l, out=(w13q, s13), out_rows=2 * H, out_row0=0)
            flow_quantize_weight(w3.detach(), E_l, out=(w13q, s13), out_rows=2 * H, out_row0=H)
            flow_quantize_weight(w2.detach(), E_l, transpose=True, out=(w2q, s2))
            self._wq_valid.add(layer)
        return w13q, s13, w2q, s2

    # -- kernels -------------------------------------------------------------------------------------
    def dispatch(self, x2, indices, slot_pos, counts_kept, scale, p_rows, epoch, p_scales=None):
        a = _lib.DispatchArgs()
        a.x, a.indices, a.slot_pos, a.counts_kept = x2.data_ptr(), indices.data_ptr(), slot_pos.data_ptr(), \
            counts_kept.data_ptr()
        a.slot_scale = scale.data_ptr() if scale is not None else None
        a.T, a.K, a.D, a.E, a.E_local, a.n_ranks, a.my_rank = self.T, self.K, self.D, self.E, self.E_local, self.N, \
            self.rank
        a.region_rows, a.quant = self.R, (2 if p_scales is not None else 0)   # 2: e4m3 + power-of-two 1x128 scales
        a.peer_rows, a.peer_scales = p_rows.data_ptr(), (p_scales.data_ptr() if p_scales is not None else None)
        a.peer_row_dst, a.peer_mblk_rows = self.p_row_dst.data_ptr(), self.p_mblk_rows.data_ptr()
        a.peer_src_blocks, a.peer_flags = self.p_src_blocks.data_ptr(), self.p_dispatch_flags.data_ptr()
        a.done_ctr, a.epoch, a.write_meta, a.max_ctas = self.dispatch_ctr.data_ptr(), epoch, 1, self.max_ctas_dispatch
        a.epoch_base = self.heap.epoch_base.data_ptr()
        _lib.check(_lib.lib().np_ep_dispatch(C.byref(a), C.c_void_p(_lib.stream())), "ep_dispatch")

    def combine(self, rows, slot_pos, weights, out, sent_to_peer, epoch, dl=None, wg=None, add1=None):
        a = _lib.CombineArgs()
        a.rows, a.slot_pos = rows.data_ptr(), slot_pos.data_ptr()
        a.weights = weights.data_ptr() if weights is not None else None
        a.add1 = add1.data_ptr() if add1 is not None else None
        a.add2 = None
        a.dl = dl.data_ptr() if dl is not None else None
        a.wg = wg.data_ptr() if wg is not None else None
        a.out = out.data_ptr()
        a.T, a.K, a.D, a.E = self.T, self.K, self.D, self.E
        a.flags, a.sent_to_peer = self.combine_flags.data_ptr(), sent_to_peer.data_ptr()
        a.n_ranks, a.epoch, a.limit_ns = self.N, epoch, WAIT_LIMIT_NS
        a.epoch_base = self.heap.epoch_base.data_ptr()
        _lib.check(_lib.lib().np_ep_combine(C.byref(a), C.c_void_p(_lib.stream())), "ep_combine")

    def grouped_gemm(self, A, B, *, N, K, b_mn, group_stride_b, out=None, B2=None, C2=None, wait_epoch=0,
                     push_ptrs=None, push_epoch=0, Cin=None, out_dtype=torch.bfloat16):
        """Row-grouped GEMM over the receive-buffer layout (mode 1)."""
        g = _lib.GemmArgs()
        M = self.rows_total
        if out is None and push_ptrs is None:
            out = torch.empty((M, N), device=A.device, dtype=out_dtype)
        g.A, g.B = A.data_ptr(), B.data_ptr()
        g.lda, g.ldb = A.stride(0), B.stride(0)
        g.a_rows, g.b_rows = A.shape[0], B.shape[0]
        g.M, g.N, g.K = M, N, K
        g.a_mn, g.b_mn = 0, int(b_mn)
        g.mode, g.alpha = 1, 1.0
        g.mblk_group, g.mblk_rows = self.mblk_group.data_ptr(), self.mblk_rows.data_ptr()
        g.group_stride_b = group_stride_b
        g.mblk_flag = self.mblk_flag.data_ptr()
        if B2 is not None:
            g.B2, g.epilogue = B2.data_ptr(), 1
            g.C2 = C2.data_ptr() if C2 is not None else None
            g.ldc2 = C2.stride(0) if C2 is not None else 0
        if wait_epoch:
            g.ready_flags, g.epoch, g.flag_limit_ns = self.dispatch_flags.data_ptr(), wait_epoch, WAIT_LIMIT_NS
        if push_ptrs is not None:
            self.done_counters.zero_()
            g.row_dst, g.peer_base = self.row_dst.data_ptr(), push_ptrs.data_ptr()
            g.done_counters, g.done_expected = self.done_counters.data_ptr(), self.src_blocks.data_ptr()
            g.done_flag_ptr, g.epoch = self.p_done_flag.data_ptr(), push_epoch
            g.C, g.ldc = None, N
            g.out_f32 = 0
        else:
            g.C, g.ldc = out.data_ptr(), out.stride(0)
            g.out_f32 = int(out.dtype == torch.float32)
        if Cin is not None:
            g.Cin, g.ldcin = Cin.data_ptr(), Cin.stride(0)
        g.epoch_base = self.heap.epoch_base.data_ptr()
        _lib.check(_lib.lib().np_gemm_bf16(C.byref(g), C.c_void_p(_lib.stream())), "grouped_gemm")
        return out

    def grouped_gemm_fp8(self, aq, sfa, bq, sfb, *, N, out=None, wait_epoch=0, push_ptrs=None, push_epoch=0):
        """Row-grouped e4m3 GEMM over the receive-buffer layout on the block-scaled tensor-core path (B K-major,
        ``N`` rows per expert; scales as exponent chunks)."""
        from .gemm_mxfp8 import gemm_mxfp8

        fill = {"mblk_flag": self.mblk_flag.data_ptr(), "epoch_base": self.heap.epoch_base.data_ptr()}
        if wait_epoch:
            fill.update(ready_flags=self.dispatch_flags.data_ptr(), epoch=wait_epoch, flag_limit_ns=WAIT_LIMIT_NS)
        if push_ptrs is not None:
            self.done_counters.zero_()
            fill.update(row_dst=self.row_dst.data_ptr(), peer_base=push_ptrs.data_ptr(),
                        done_counters=self.done_counters.data_ptr(), done_expected=self.src_blocks.data_ptr(),
                        done_flag_ptr=self.p_done_flag.data_ptr(), epoch=push_epoch)
        return gemm_mxfp8(aq, sfa, bq, sfb, out=out, mblk_group=self.mblk_group, mblk_rows=self.mblk_rows,
                          rows_per_group=N, fill=fill)

    def grouped_wgrad(self, A, Bm, w: torch.Tensor, *, M, N):
        """dW[g] (+)= A[rows of g]^T @ B[rows of g] for every local expert g (mode 2), into ``main_grad``
        when the weight has one, else a fresh tensor that is returned."""
        mg = getattr(w, "main_grad", None)
        first = not getattr(w, "_main_grad_dirty", False)
        out = mg if mg is not None else torch.empty((self.E_local * M, N), device=A.device, dtype=torch.float32)
        g = _lib.GemmArgs()
        g.A, g.B, g.C = A.data_ptr(), Bm.data_ptr(), out.data_ptr()
        g.lda, g.ldb, g.ldc = A.stride(0), Bm.stride(0), N
        g.a_rows, g.b_rows = A.shape[0], Bm.shape[0]
        g.M, g.N, g.K = M, N, self.rows_total
        g.a_mn, g.b_mn, g.mode, g.alpha = 1, 1, 2, 1.0
        g.out_f32 = 1
        g.accumulate = int(mg is not None and not first)
        g.mblk_rows = self.mblk_rows.data_ptr()
        g.num_groups, g.blocks_per_group, g.group_stride_c = self.E_local, self.N * self.bpr, M * N
        _lib.check(_lib.lib().np_gemm_bf16(C.byref(g), C.c_void_p(_lib.stream())), "grouped_wgrad")
        if mg is not None:
            w._main_grad_dirty = True
            return None
        return out.to(w.dtype)


# ------------------------------------------------------------------------------------------------ the layer
class _FusedMoE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weights, indices32, w1, w3, w2, rt: FusedMoERuntime, layer: int, stats_mod, shared=None):
        T, D, K, H = rt.T, rt.D, rt.K, rt.H
        dev = x.device
        x2 = x.reshape(T, D)
        x2 = x2 if x2.is_contiguous() else x2.contiguous()
        slot_pos = torch.empty((T, K), device=dev, dtype=torch.int32)
        keep = torch.empty(T, device=dev, dtype=torch.int32)
        counts_kept = torch.empty(rt.E, device=dev, dtype=torch.int32)
        drops = torch.empty(rt.E, device=dev, dtype=torch.int32)
        n_dropped = torch.empty(1, device=dev, dtype=torch.int32)
        _lib.call("capacity_scan", indices32, T, rt.E, K, rt.capacity, slot_pos, keep, counts_kept, drops, n_dropped)
        sent = counts_kept.view(rt.N, rt.E_local).sum(1).to(torch.int32)
        e1 = rt.next_epoch()
        gu = torch.empty((rt.rows_total, 2 * H), device=dev, dtype=torch.bfloat16)
        if rt.fp8:
            # FP8-Flow-MoE forward: rows travel as e4m3 with 1x128 power-of-two scales (quantised inside the dispatch
            # kernel), the expert weights are e4m3 with 128x128 scales (made once per optimizer step), both expert
            # GEMMs run on the block-scaled tcgen05 path with the scaling done by the tensor core: one gate|up GEMM,
            # SwiGLU + re-quantisation in one pass, and the down GEMM pushing rows back to their sources
            from .gemm_mxfp8 import flow_quantize_act

            w13q, s13, w2q, s2 = rt.quantised_weights(layer, w1, w3, w2)
            rt.dispatch(x2, indices32, slot_pos, counts_kept, None, rt.p_recv_xq[layer], e1,
                        p_scales=rt.p_recv_xs[layer])
            xq, xs = rt.recv_xq[layer].view(torch.float8_e4m3fn), rt.recv_xs[layer]
            rt.grouped_gemm_fp8(xq, xs, w13q, s13, N=2 * H, out=gu, wait_epoch=e1)
            h = torch.empty((rt.rows_total, H), device=dev, dtype=torch.bfloat16)
            hq, hs = flow_quantize_act(gu, swiglu=True, h_out=h)
            rt.grouped_gemm_fp8(hq, hs, w2q, s2, N=D, push_ptrs=rt.p_ret_y[layer], push_epoch=e1)
        else:
            rt.dispatch(x2, indices32, slot_pos, counts_kept, None, rt.p_recv_x[layer], e1)
            # experts: [gate|up] GEMM with SwiGLU epilogue, waits per block on the source's arrival flag
            h = torch.empty((rt.rows_total, H), device=dev, dtype=torch.bfloat16)
            rt.grouped_gemm(rt.recv_x[layer], w1, N=H, K=D, b_mn=False, group_stride_b=H, out=h, B2=w3, C2=gu,
                            wait_epoch=e1)
            # down projection (w2 is stored [H, D] per expert: MN-major B), rows pushed back to their sources
            rt.grouped_gemm(h, w2, N=D, K=H, b_mn=True, group_stride_b=H, push_ptrs=rt.p_ret_y[layer],
                            push_epoch=e1)
        out = torch.empty((T, D), device=dev, dtype=torch.bfloat16)
        add1 = None
        if shared is not None:
            # the shared expert's output joins in the combine pass; a token dropped by the capacity rule gets no
            # MoE output at all, shared expert included (reference: model/moe.py:1383-1390)
            add1 = shared.reshape(T, D) * keep.to(shared.dtype).unsqueeze(1)
        rt.combine(rt.ret_y[layer], slot_pos, weights, out, sent, e1, add1=add1)
        ctx.has_shared = shared is not None
        # the activation h is kept for the w2 weight gradient (57 MB per layer at the 1B shapes: cheap next to
        # re-reading the pre-activations)
        ctx.has_h = True
        ctx.save_for_backward(x2, weights, indices32, slot_pos, counts_kept, sent, gu, w1, w3, w2,
                              *([h] if ctx.has_h else []), *([keep] if ctx.has_shared else []))
        ctx.rt, ctx.layer = rt, layer
        ctx.x_shape = x.shape
        if stats_mod is not None:
            stats_mod._per_expert_drop_counts = drops
            stats_mod._record_drops(n_dropped[0].long(), T, dev)
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, dout):
        x2, weights, indices32, slot_pos, counts_kept, sent, gu, w1, w3, w2 = ctx.saved_tensors[:10]
        rt, layer = ctx.rt, ctx.layer
        T, D, K, H = rt.T, rt.D, rt.K, rt.H
        dev = dout.device
        do2 = dout.reshape(T, D)
        do2 = do2 if do2.is_contiguous() else do2.contiguous()
        # d(router weights)[t,k] = <dout[t], y[t,k]>
        dweights = torch.empty((T, K), device=dev, dtype=torch.float32)
        _lib.call("slot_dot", do2, rt.ret_y[layer], slot_pos, dweights, T, K, D)
        # send w[t,k] * dout[t] to the experts (same slots as forward)
        e2 = rt.next_epoch()
        rt.dispatch(do2, indices32, slot_pos, counts_kept, weights, rt.p_recv_g, e2)
        # dH = dY @ w2^T  (w2 [H, D] per expert is K-major for this contraction)
        dh = rt.grouped_gemm(rt.recv_g, w2, N=H, K=D, b_mn=False, group_stride_b=H, wait_epoch=e2)
        hh = ctx.saved_tensors[10] if ctx.has_h else glu(gu)
        dw2 = rt.grouped_wgrad(hh, rt.recv_g, w2, M=H, N=D)
        del hh
        dgu = glu_bwd(gu, dh)
        del dh
        dg, du = dgu[:, :H], dgu[:, H:]
        if rt.fp8:  # the rows arrived as e4m3: dequantise once for the (bf16) weight-gradient GEMMs
            from .gemm_mxfp8 import mx_dequantize_bf16

            xr = mx_dequantize_bf16(rt.recv_xq[layer].view(torch.float8_e4m3fn), rt.recv_xs[layer])
        else:
            xr = rt.recv_x[layer]
        dw1 = rt.grouped_wgrad(dg, xr, w1, M=H, N=D)
        dw3 = rt.grouped_wgrad(du, xr, w3, M=H, N=D)
        # dX = dG @ w1 + dU @ w3, pushed back to the sources
        part = rt.grouped_gemm(dg, w1, N=D, K=H, b_mn=True, group_stride_b=H)
        rt.grouped_gemm(du, w3, N=D, K=H, b_mn=True, group_stride_b=H, push_ptrs=rt.p_ret_g, push_epoch=e2, Cin=part)
        dx = torch.empty((T, D), device=dev, dtype=torch.bfloat16)
        rt.combine(rt.ret_g, slot_pos, None, dx, sent, e2)
        dshared = None
        if ctx.has_shared:
            keep = ctx.saved_tensors[-1]
            dshared = (do2 * keep.to(do2.dtype).unsqueeze(1)).view(ctx.x_shape)
        return dx.view(ctx.x_shape), dweights, None, dw1, dw3, dw2, None, None, None, dshared


def build_runtime(moe_modules, *, tokens: int, group=None, device=None) -> FusedMoERuntime:
    """One runtime for all MoE layers of a model (they must share geometry)."""
    import torch.distributed as dist

    m0 = moe_modules[0]
    world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
    # FP8-Flow-MoE switch: fp8 expert GEMMs once the expected tokens per expert reach the threshold
    per_expert = tokens * m0.top_k * world / m0.num_experts
    # ("fp8 grouped GEMM above N tokens per expert and bf16 below": strictly above)
    fp8 = bool(m0.fp8_flow_moe_enabled and m0.fp8_recipe in ("blockwise", "flow_moe") and
               per_expert > m0.fp8_gemm_threshold)
    disp = getattr(m0.ep, "dispatcher", None)
    max_ctas = 0
    if hasattr(disp, "dispatch_ctas"):      # DeepEPDispatcher knobs: SM budget of the dispatch kernel, e4m3 on the wire
        fp8 = fp8 or bool(getattr(disp, "use_fp8_dispatch", False))
        max_ctas = disp.dispatch_ctas(tokens=tokens, d_model=m0.d_model, hidden=m0.hidden_size,
                                      num_experts=m0.num_experts, top_k=m0.top_k, fp8=fp8)
    rt = FusedMoERuntime(tokens=tokens, d_model=m0.d_model, hidden=m0.hidden_size, num_experts=m0.num_experts,
                         top_k=m0.top_k, n_layers=len(moe_modules), capacity_factor=m0.capacity_factor, group=group,
                         device=device, fp8=fp8, max_ctas_dispatch=max_ctas)
    for m in moe_modules:
        m._fused_runtime = rt
        rt.layer_index(m)
    if m0.router.score_bias is not None:
        rt.bind_router_bias(moe_modules)
    return rt


def fused_moe_forward(mod, x: torch.Tensor) -> torch.Tensor:
    """Forward of ``MoEBase`` on the fused path (``x``: [B, S, D] bf16 on CUDA)."""
    rt: FusedMoERuntime = mod._fused_runtime
    B, S, D = x.shape
    if B * S != rt.T or mod.capacity_factor is not None and int(mod.capacity_factor * B * S / mod.num_experts) != \
            rt.capacity:
        raise _lib.KernelError(f"fused MoE runtime was built for {rt.T} tokens / capacity {rt.capacity}; got "
                               f"{B * S} tokens (rebuild the runtime or call the layer with a matching batch)")
    cfg = mod.router.config
    xr = x
    if cfg.jitter_eps is not None and mod.training:   # routing noise, as in MoERouter.forward
        xr = x + torch.randn_like(x) * cfg.jitter_eps
    w, idx, aux, counts = route(xr, mod.router)
    mod.router.last_counts = counts
    layer = rt.layer_index(mod)
    if mod.router.score_bias is not None:
        if rt.score_bias_all is not None:
            rt.bias_counts[layer].add_(counts)
        else:
            mod.router._update_expert_counts(idx, counts)
    mod._aux_loss = aux
    shared = mod.shared_expert(x) if mod.shared_expert is not None else None
    with _lib.nvtx_range("fused_moe"):
        return _FusedMoE.apply(x, w.reshape(B * S, -1), idx.reshape(B * S, -1).to(torch.int32), mod.w1, mod.w3,
                               mod.w2, rt, layer, mod, shared)
