"""Flat parameter arena and the fused AdamW that runs on it.

All parameters of a model are re-pointed into a few flat buffers ("regions": bf16 replicated, bf16
expert-sharded, fp32), each with a flat fp32 gradient buffer (``param.main_grad`` views) and flat
fp32 master / moment buffers. That layout is what the B200 kernels want:

* adjacent weights become one GEMM operand without a copy (``[w_q|w_k|w_v]``, ``[w1;w3]``);
* wgrad GEMMs accumulate straight from TMEM into ``main_grad`` (no autograd ``.grad`` tensors);
* the optimizer is one launch per region, reading the gradient once and writing the bf16 weights in
  the same pass; gradient clipping uses device-side partial sums, no host synchronisation;
* with data parallelism the replicated bf16 region lives in symmetric memory and the step becomes
  reduce-scatter (peer loads) -> AdamW on the owned shard -> all-gather (peer stores), two launches
  (``csrc/comm.cu``), with optimizer state sharded over the ranks (ZeRO-2 layout).

The reference uses ``torch.optim.AdamW`` on autocast fp32 weights (cli.py:356-361) or its per-tensor
Python loop (optim/adamw.py:74-121), FSDP2 for sharding and ``clip_grad_norm_`` (trainer.py:280-284).
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from ..ops import _lib
from .adamw import is_no_decay

ALIGN = 64  # elements; keeps every view 128-byte aligned


@dataclass
class _Region:
    name: str
    dtype: torch.dtype
    decay: bool
    replicated: bool            # True: identical on all data-parallel ranks (needs gradient sync)
    params: List[nn.Parameter] = field(default_factory=list)
    names: List[str] = field(default_factory=list)
    offsets: List[int] = field(default_factory=list)
    numel: int = 0
    weights: Optional[torch.Tensor] = None   # flat, region dtype
    grads: Optional[torch.Tensor] = None     # flat fp32
    master: Optional[torch.Tensor] = None    # flat fp32 (shard under ZeRO); None for fp32 regions
    m: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    lo: int = 0                              # owned shard [lo, lo+cnt) under ZeRO
    cnt: int = 0
    gshard: Optional[torch.Tensor] = None
    tp_group: Optional[object] = None        # tensor-parallel group these parameters are shards over (None: whole)
    sp_group: Optional[object] = None        # group over which these parameters' gradients are partial sums (whole
    #                                          parameters applied to row shards under sequence parallelism)
    # overlapped reduce-scatter (ZeRO regions): the flat buffer is cut into equal buckets, rank r owns slice r of every
    # bucket; master / m / v / gshard hold the owned slices back to back in bucket order
    bucket: int = 0                          # elements per bucket (0: one contiguous shard, no overlap)
    slice: int = 0                           # bucket // world
    n_buckets: int = 0
    pending: Optional[List[int]] = None      # per bucket: parameters whose gradient is still to come this step
    need: Optional[List[int]] = None         # per bucket: number of parameters overlapping it
    launched: Optional[List[bool]] = None
    flags: Optional[torch.Tensor] = None     # symmetric int32 [n_buckets * world]
    staged: Optional[torch.Tensor] = None    # copy mode: [(world - 1) * cnt] peer slices in the compact shard order
    mc_weights: int = 0                      # NVLink multicast addresses of the weight / gradient arenas (0: none)
    mc_grads: int = 0
    _mc_keep: Optional[tuple] = None         # symmetric-memory handles, kept alive with the region


def owned_slice(flat: torch.Tensor, world: int, rank: int, bucket: int) -> torch.Tensor:
    """Rank ``rank``'s part of a flat region buffer of a ``world``-way sharded arena: one contiguous piece, or - with
    the bucketed reduce-scatter - slice ``rank`` of every bucket, back to back."""
    if bucket:
        return flat.view(-1, world, bucket // world)[:, rank].reshape(-1)
    cnt = flat.numel() // world
    return flat[rank * cnt:(rank + 1) * cnt]


def assemble_shards(shards: List[torch.Tensor], bucket: int) -> torch.Tensor:
    """Inverse of ``owned_slice``: the flat buffer from the parts of all ranks (in rank order)."""
    world = len(shards)
    if bucket:
        sl = bucket // world
        return torch.stack([sh.view(-1, sl) for sh in shards], dim=1).reshape(-1)
    return torch.cat(shards)


class ParamArena:
    def __init__(self, model: nn.Module, *, dp_group=None, device=None, use_symmetric: Optional[bool] = None,
                 bucket_elems: Optional[int] = None, replicate_group=None, expert_replica_group=None):
        params = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        assert params, "model has no trainable parameters"
        self.model = model
        self.device = device or params[0][1].device
        self.dp_group = dp_group
        self.world = dist.get_world_size(dp_group) if (dp_group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(dp_group) if self.world > 1 else 0
        # hybrid sharding (HSDP): optimizer state and gradients are sharded over ``dp_group`` and every shard is
        # replicated over ``replicate_group``; reduced gradient shards are summed across the replicas before the update
        self.replicate_group = replicate_group
        self.rep_world = dist.get_world_size(replicate_group) if (replicate_group is not None and
                                                                  dist.is_initialized()) else 1
        # ranks holding a copy of the same expert shard that see other tokens (ep_size below the data-parallel size):
        # the gradients of the expert-sharded regions are summed over them before the update
        self.expert_replica_group = expert_replica_group
        self.expert_rep_world = dist.get_world_size(expert_replica_group) if (
            expert_replica_group is not None and dist.is_initialized()) else 1
        cuda = self.device.type == "cuda"
        self.zero = self.world > 1 and cuda if use_symmetric is None else bool(use_symmetric)
        import os as _os

        if bucket_elems is None:
            env = _os.environ.get("NPB200_ZERO_BUCKET")
            if env is not None:
                bucket_elems = int(env)
            else:
                # With expert parallelism over more than two GPUs the bulk copies of the overlapped reduction share the
                # NVLink ports with the dispatch / combine pushes that the expert GEMMs wait for: measured on the 1B
                # MoE step, 8 GPUs, 31.3 ms with the overlap against 30.3 ms without (2 GPUs: 34.0 against 34.3).
                has_ep = any(getattr(p_, "_ep_sharded", False) for p_ in model.parameters())
                bucket_elems = 0 if (has_ep and self.world > 2) else (16 << 20)
        q = 4 * self.world * ALIGN
        self.bucket_elems = 0 if (bucket_elems <= 0 or _os.environ.get("NPB200_NVLS", "0") == "1") else \
            (bucket_elems + q - 1) // q * q
        # Overlapped reduce-scatter: while the backward pass runs, the copy engines fetch the peers' slices of every
        # finished bucket (cudaMemcpyAsync over NVLink) into a staging buffer, one kernel sums them afterwards. No SM is
        # taken from the GEMMs. (A small pulling kernel per bucket on a side stream was measured first: its CTAs share
        # SMs with the persistent GEMM CTAs and slow them; 38.2 ms per step against 34.2 without overlap on 2 GPUs.)
        self.reduce_enabled = True      # False while earlier micro-batches of an accumulation step run
        self._late_write = False
        self._side: Optional[torch.cuda.Stream] = torch.cuda.Stream(device=self.device) if (self.zero and cuda) else None
        self._epoch = 0
        self.regions: Dict[str, _Region] = {}
        seen = set()
        for n, p in self._gate_up_adjacent(params):
            if id(p) in seen:
                continue
            seen.add(id(p))
            sharded = bool(getattr(p, "_ep_sharded", False))
            tpg = getattr(p, "_tp_sharded", None)
            spg = getattr(p, "_sp_reduce_group", None)
            decay = not is_no_decay(n, p)
            key = f"{str(p.dtype).split('.')[-1]}_{'local' if sharded else 'repl'}_{'decay' if decay else 'nodecay'}" \
                  f"{'_tp' if tpg is not None else ''}{'_sp' if spg is not None else ''}"
            r = self.regions.setdefault(key, _Region(key, p.dtype, decay, not sharded, tp_group=tpg, sp_group=spg))
            off = (r.numel + ALIGN - 1) // ALIGN * ALIGN if not self._adjacent_ok(r, p) else r.numel
            r.params.append(p)
            r.names.append(n)
            r.offsets.append(off)
            r.numel = off + p.numel()
        self.heap = None
        # scale of the reduced gradients (set by the optimizer every step)
        self.grad_inv = 1.0 / (max(self.world, 1) * max(self.rep_world, 1))
        if self.zero:
            from ..parallel.symm import SymmetricHeap

            need = 0
            for r in self.regions.values():
                if r.replicated and r.dtype == torch.bfloat16:
                    pad = self._padded(r.numel)
                    need += pad * 2 + pad * 4 + 8192 + 4 * self.world * (pad // max(self.bucket_elems, 1) + 2)
            f32_elems = sum(r.numel for r in self.regions.values() if r.replicated and r.dtype == torch.float32)
            self._ar_max = max(f32_elems + 64, 4096)
            self.heap = SymmetricHeap(need + 2 * self.world * self._ar_max * 4 + (1 << 20), dp_group, self.device)
            self.heap.reserve_allreduce(self._ar_max)
        self.fused: List[torch.Tensor] = []
        for r in self.regions.values():
            self._materialise(r)
        self._install_hooks()
        self._fuse_views()

    # ------------------------------------------------------------------ construction
    @staticmethod
    def _gate_up_adjacent(params):
        """The layout order: the model's parameter order, except that a feed-forward's up projection ``w3.weight``
        follows its gate projection ``w1.weight`` directly (the module registers w1, w2, w3), so that ``_fuse_views`` can
        hand the layer one ``[w1; w3]`` matrix for a single gate|up GEMM."""
        by_name = dict(params)
        out, done = [], set()
        for n, p in params:
            if n in done:
                continue
            out.append((n, p))
            done.add(n)
            if n.endswith("w1.weight"):
                partner = n[:-len("w1.weight")] + "w3.weight"
                if partner in by_name and partner not in done:
                    out.append((partner, by_name[partner]))
                    done.add(partner)
        return out

    @staticmethod
    def _adjacent_ok(r: _Region, p) -> bool:
        # sizes that are multiples of ALIGN keep alignment without padding, so neighbours stay adjacent
        return r.numel % ALIGN == 0

    def _padded(self, n: int) -> int:
        q = self.bucket_elems if (self.zero and self.bucket_elems) else 4 * self.world * ALIGN
        return (n + q - 1) // q * q

    def _materialise(self, r: _Region):
        dev = self.device
        symm = self.zero and r.replicated and r.dtype == torch.bfloat16
        total = self._padded(r.numel) if symm else (r.numel + 3) // 4 * 4
        if symm:
            from ..parallel.symm import nvls_alloc

            # NVLS: both arenas in multicast-bound memory, so that the gradient reduction happens inside the switch
            # and one store delivers the new weights to every rank; otherwise plain peer loads / stores
            mw = nvls_alloc(total, r.dtype, self.dp_group, dev)
            mg = nvls_alloc(total, torch.float32, self.dp_group, dev) if mw is not None else None
            if mw is not None and mg is not None:
                r.weights, r.mc_weights, r._mc_keep = mw[0], mw[1], (mw[2], mg[2])
                r.grads, r.mc_grads = mg[0], mg[1]
                r.weights.zero_()
                r.grads.zero_()
            else:
                r.weights = self.heap.alloc((total,), r.dtype)
                r.grads = self.heap.alloc((total,), torch.float32)
            r.cnt = total // self.world
            r.lo = self.rank * r.cnt
            if self.bucket_elems and not r.mc_grads:
                r.bucket, r.slice, r.n_buckets = self.bucket_elems, self.bucket_elems // self.world, \
                    total // self.bucket_elems
                r.lo = self.rank * r.slice
                r.flags = self.heap.alloc((r.n_buckets * self.world,), torch.int32)
                r.staged = torch.empty((self.world - 1) * r.cnt, device=dev, dtype=torch.float32)
        else:
            r.weights = torch.zeros(total, device=dev, dtype=r.dtype)
            r.grads = torch.zeros(total, device=dev, dtype=torch.float32)
            r.lo, r.cnt = 0, total
        with torch.no_grad():
            for p, off in zip(r.params, r.offsets):
                view = r.weights[off:off + p.numel()].view(p.shape)
                view.copy_(p.data)
                p.data = view
                p.main_grad = r.grads[off:off + p.numel()].view(p.shape)
                p._main_grad_dirty = False
        if r.dtype != torch.float32:
            r.master = self.owned(r, r.weights).float()
        r.m = torch.zeros(r.cnt, device=dev, dtype=torch.float32)
        r.v = torch.zeros(r.cnt, device=dev, dtype=torch.float32)
        if symm:
            r.gshard = torch.empty(r.cnt, device=dev, dtype=torch.float32)

    def owned(self, r: _Region, flat: torch.Tensor) -> torch.Tensor:
        """This rank's part of a flat region buffer, in the order master / m / v / gshard hold it."""
        if r.bucket:
            return flat.view(r.n_buckets, self.world, r.slice)[:, self.rank].reshape(-1)
        return flat[r.lo:r.lo + r.cnt]

    def _install_hooks(self):
        def hook(p):
            if p.grad is None:
                return
            if getattr(p, "_main_grad_dirty", False):
                p.main_grad.add_(p.grad)
            else:
                p.main_grad.copy_(p.grad)
                p._main_grad_dirty = True
            p.grad = None
            cb = getattr(p, "_grad_ready_cb", None)
            if cb is not None:
                cb(p)

        for r in self.regions.values():
            for p in r.params:
                p.register_post_accumulate_grad_hook(hook)
            if r.bucket:
                # which buckets each parameter overlaps; a bucket is reduced as soon as all of them have their gradient
                r.need = [0] * r.n_buckets
                for p, off in zip(r.params, r.offsets):
                    bs = list(range(off // r.bucket, (off + p.numel() - 1) // r.bucket + 1))
                    p._arena_buckets = (r, bs)
                    p._grad_ready_cb = self._param_ready
                    for b in bs:
                        r.need[b] += 1
                r.pending = list(r.need)
                r.launched = [False] * r.n_buckets

    # ------------------------------------------------------------------ overlapped gradient reduction
    def _param_ready(self, p):
        """Called when a parameter's gradient for this backward pass has been written (wgrad GEMM epilogue,
        embedding backward kernel or the autograd hook above)."""
        if not self.reduce_enabled:
            return
        if getattr(p, "_arena_counted", False):
            if any(p._arena_buckets[0].launched[b] for b in p._arena_buckets[1]):
                self._late_write = True      # a second backward wrote after the bucket went out: redone in step()
            return
        p._arena_counted = True
        r, bs = p._arena_buckets
        for b in bs:
            r.pending[b] -= 1
            if r.pending[b] == 0 and not r.launched[b]:
                self._launch_bucket(r, b)

    def _launch_bucket(self, r: _Region, b: int):
        import ctypes as C

        if not any(x for rr in self.regions.values() if rr.bucket for x in rr.launched):
            self._epoch = self.heap.next_epoch()      # one epoch per step for every bucket flag
        main = torch.cuda.current_stream()
        self._side.wait_stream(main)
        with torch.cuda.stream(self._side):
            lo = b * r.bucket + self.rank * r.slice
            lib, st = _lib.lib(), C.c_void_p(_lib.stream())
            _lib.check(lib.np_bucket_sync(self.heap.host_ptr_array(r.flags), b, self.rank, self.world, self._epoch,
                                          C.c_void_p(self.heap.epoch_base.data_ptr()), C.c_ulonglong(0), st),
                       "bucket_sync")
            k = 0
            for peer in range(self.world):
                if peer == self.rank:
                    continue
                src = self.heap.peer_ptr(r.grads, peer) + lo * 4
                dstp = r.staged.data_ptr() + (k * r.cnt + b * r.slice) * 4
                _lib.check(lib.np_memcpy_async(C.c_void_p(dstp), C.c_void_p(src), C.c_ulonglong(r.slice * 4), st),
                           "memcpy_async")
                k += 1
        r.launched[b] = True

    def finish_buckets(self):
        """Launch whatever has not gone out yet (parameters without a gradient this step were just zeroed), redo
        everything if a later backward pass wrote into a bucket that had already been reduced, and make the current
        stream wait for the side stream."""
        regs = [r for r in self.regions.values() if r.bucket]
        if not regs:
            return
        if self._late_write:
            if self._side is not None:
                torch.cuda.current_stream().wait_stream(self._side)
            for r in regs:
                r.launched = [False] * r.n_buckets
            self._late_write = False
        for r in regs:
            for b in range(r.n_buckets):
                if not r.launched[b]:
                    self._launch_bucket(r, b)
        torch.cuda.current_stream().wait_stream(self._side)

    def reset_buckets(self):
        for r in self.regions.values():
            if r.bucket:
                r.pending = list(r.need)
                r.launched = [False] * r.n_buckets
                for p in r.params:
                    p._arena_counted = False

    def _region_of(self, p) -> Optional[tuple]:
        for r in self.regions.values():
            for q, off in zip(r.params, r.offsets):
                if q is p:
                    return r, off
        return None

    def _fused_view(self, plist) -> Optional[torch.Tensor]:
        """One [sum rows, cols] view over parameters that sit back to back in a region."""
        loc = [self._region_of(p) for p in plist]
        if any(l is None for l in loc) or len({id(l[0]) for l in loc}) != 1:
            return None
        r = loc[0][0]
        off0, cols, end = loc[0][1], plist[0].shape[1], loc[0][1]
        for p, (_, off) in zip(plist, loc):
            if off != end or p.dim() != 2 or p.shape[1] != cols:
                return None
            end = off + p.numel()
        rows = sum(p.shape[0] for p in plist)
        w = r.weights[off0:end].view(rows, cols)
        w.main_grad = r.grads[off0:end].view(rows, cols)
        w._main_grad_dirty = False
        w._covers = list(plist)
        recipes = {getattr(p, "_fp8_recipe", None) for p in plist}
        if len(recipes) == 1 and None not in recipes:  # all covered weights share an fp8 recipe
            w._fp8_recipe = recipes.pop()
        self.fused.append(w)
        return w

    def _fuse_views(self):
        from ..models.attention import Attention
        from ..models.feed_forward import FeedForward

        if self.device.type != "cuda":
            return
        for m in self.model.modules():
            if any(hasattr(p, "_fsdp_rt") for p in m.parameters(recurse=False)) or \
                    any(hasattr(l.weight, "_fsdp_rt") for l in m.children() if isinstance(l, nn.Linear)):
                continue  # row-sharded weights are gathered one by one inside their GEMMs
            if isinstance(m, Attention) and m.w_q.bias is None and m.w_q.weight.dtype == torch.bfloat16:
                m._fused_qkv = self._fused_view([m.w_q.weight, m.w_k.weight, m.w_v.weight])
            elif isinstance(m, FeedForward) and m.w1.bias is None and m.w1.weight.dtype == torch.bfloat16:
                m._fused_w13 = self._fused_view([m.w1.weight, m.w3.weight])

    # ------------------------------------------------------------------ per-step helpers
    def zero_grad(self):
        """Marks every gradient buffer as "overwrite on first write"; nothing is memset."""
        for r in self.regions.values():
            for p in r.params:
                p._main_grad_dirty = False
                p.grad = None
        for w in self.fused:
            w._main_grad_dirty = False
        self.reset_buckets()

    def finalize_grads(self):
        """Zero the gradient of any parameter that received none this step."""
        for r in self.regions.values():
            for p in r.params:
                if not p._main_grad_dirty:
                    p.main_grad.zero_()

    def num_params(self) -> int:
        return sum(p.numel() for r in self.regions.values() for p in r.params)

    def named_main_grads(self):
        for r in self.regions.values():
            for n, p in zip(r.names, r.params):
                yield n, p.main_grad


class ArenaAdamW(torch.optim.Optimizer):
    """AdamW over a ``ParamArena`` (one fused launch per region; ZeRO kernels under data parallelism).

    ``grad_divisor`` divides every gradient before clipping (number of data-parallel ranks times
    gradient-accumulation steps when the per-rank loss is already a mean)."""

    def __init__(self, arena: ParamArena, lr: float = 3e-4, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.1, max_grad_norm: Optional[float] = 1.0, grad_divisor: float = 1.0):
        self.arena = arena
        allp = [p for r in arena.regions.values() for p in r.params]
        super().__init__([{"params": allp}], dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.max_grad_norm = max_grad_norm
        self.grad_divisor = grad_divisor
        self.step_count = 0
        # process groups over which the squared gradient norm is additionally summed before clipping (pipeline stages
        # hold disjoint parameters: the PP group), and how many ranks of those groups hold every parameter (DualPipe: 2)
        self.norm_groups: list = []
        self.norm_copies: float = 1.0
        # second stream of the two-stream parameter update (created here: not inside a graph capture)
        self._side2: Optional[torch.cuda.Stream] = torch.cuda.Stream(device=arena.device) \
            if (arena.zero and arena.device.type == "cuda") else None
        dev = arena.device
        self._cuda = dev.type == "cuda"
        nreg = len(arena.regions)
        if self._cuda:
            self._parts = _lib.lib().np_sumsq_parts()
            zp = _lib.lib().np_zero_parts()
            self._partial = torch.zeros(nreg * max(self._parts, zp), device=dev, dtype=torch.float32)
        # [lr, 1 - b1^t, 1 - b2^t]: read by the kernels from device memory so a captured step replays
        # with the current schedule; refreshed by ``update_hyper()`` (a pinned-host -> device copy)
        self._hyper = torch.zeros(3, device=dev, dtype=torch.float32)
        self._hyper_host = torch.zeros(3, dtype=torch.float32).pin_memory() if self._cuda else torch.zeros(3)
        self.post_step_hooks = []  # callables run at the end of every step (e.g. epoch bookkeeping)
        self._tot = torch.zeros(1, device=dev, dtype=torch.float32)
        self._tot2 = torch.zeros(2, device=dev, dtype=torch.float32)
        self._coef = torch.ones(2, device=dev, dtype=torch.float32)   # [clip coefficient, grad norm]
        self._coef_local = torch.ones(1, device=dev, dtype=torch.float32)
        self.last_grad_norm: Optional[torch.Tensor] = None

    @property
    def grad_divisor(self) -> float:
        return self._grad_divisor

    @grad_divisor.setter
    def grad_divisor(self, v: float):
        # the overlapped bucket reductions run during the backward pass, before step(): they read the scale here
        self._grad_divisor = float(v)
        a = self.arena
        a.grad_inv = 1.0 / (self._grad_divisor * (a.world if a.world > 1 else 1) * max(a.rep_world, 1))

    def zero_grad(self, set_to_none: bool = True):
        self.arena.zero_grad()

    # ------------------------------------------------------------------ step
    def update_hyper(self, advance: bool = True):
        """Advance the step counter and publish lr / bias corrections to the device buffer. ``step()``
        does this itself; a captured graph replays ``step(_hyper_ready=True)`` after calling this."""
        if advance:
            self.step_count += 1
        g = self.param_groups[0]
        b1, b2 = g["betas"]
        self._hyper_host[0] = g["lr"]
        self._hyper_host[1] = 1.0 - b1 ** self.step_count
        self._hyper_host[2] = 1.0 - b2 ** self.step_count
        self._hyper.copy_(self._hyper_host, non_blocking=True)

    @torch.no_grad()
    def step(self, closure=None, _hyper_ready: bool = False):
        with _lib.nvtx_range("optimizer.step"):
            return self._step(_hyper_ready)

    def _step(self, _hyper_ready: bool = False):
        a = self.arena
        a.finalize_grads()
        if not _hyper_ready:
            self.update_hyper()
        g = self.param_groups[0]
        lr, (b1, b2), eps, wd = g["lr"], g["betas"], g["eps"], g["weight_decay"]
        if not self._cuda:
            return self._step_reference(lr, b1, b2, eps, wd)
        N = a.world
        R = a.rep_world
        inv = 1.0 / (self.grad_divisor * (N if N > 1 else 1) * R)
        stride = self._partial.numel() // len(a.regions)
        self._partial.zero_()
        bucketed = a.zero and any(r.bucket for r in a.regions.values())
        if bucketed:
            # the reduce-scatter of every bucket was launched on the side stream while the backward pass ran (each
            # waits on per-bucket flags of all ranks): send the stragglers and join
            a.finish_buckets()
        if a.zero and any(r.replicated and r.dtype == torch.bfloat16 and not r.bucket for r in a.regions.values()):
            a.heap.barrier()  # every rank's backward has finished writing its gradient buffers
        extra = None
        for i, r in enumerate(a.regions.values()):
            part = self._partial[i * stride:(i + 1) * stride]
            if r.bucket:
                _lib.check(_lib.lib().np_zero_reduce_staged(
                    C.c_void_p(r.grads.data_ptr()), C.c_longlong(r.lo), C.c_longlong(r.slice), C.c_longlong(r.bucket),
                    C.c_void_p(r.staged.data_ptr()), N - 1, C.c_longlong(r.cnt), C.c_float(inv),
                    C.c_void_p(r.gshard.data_ptr()), C.c_void_p(part.data_ptr()), C.c_void_p(_lib.stream())),
                    "zero_reduce_staged")
                if R > 1 or r.sp_group is not None:   # HSDP: sum the shard over the replicas, then take its norm
                    if R > 1:
                        dist.all_reduce(r.gshard, group=a.replicate_group)
                    if r.sp_group is not None:
                        dist.all_reduce(r.gshard, group=r.sp_group)
                    part.zero_()
                    _lib.call("sumsq", r.gshard, _lib.LL(r.gshard.numel()), part)
            elif a.zero and r.replicated and r.dtype == torch.bfloat16 and r.mc_grads:
                _lib.check(_lib.lib().np_zero_reduce_mc(C.c_void_p(r.mc_grads), C.c_longlong(r.lo), C.c_longlong(r.cnt),
                                                        C.c_float(inv), C.c_void_p(r.gshard.data_ptr()),
                                                        C.c_void_p(part.data_ptr()), C.c_void_p(_lib.stream())),
                           "zero_reduce_mc")
            elif a.zero and r.replicated and r.dtype == torch.bfloat16:
                ptrs = a.heap.host_ptr_array(r.grads)
                _lib.check(_lib.lib().np_zero_reduce(ptrs, N, C.c_longlong(r.lo), C.c_longlong(r.cnt),
                                                     C.c_float(inv), C.c_void_p(r.gshard.data_ptr()),
                                                     C.c_void_p(part.data_ptr()), C.c_void_p(_lib.stream())),
                           "zero_reduce")
                if R > 1 or r.sp_group is not None:
                    if R > 1:
                        dist.all_reduce(r.gshard, group=a.replicate_group)
                    if r.sp_group is not None:
                        dist.all_reduce(r.gshard, group=r.sp_group)
                    part.zero_()
                    _lib.call("sumsq", r.gshard, _lib.LL(r.gshard.numel()), part)
            else:
                if N > 1 and r.replicated:  # small fp32 region: all-reduce through peer memory (NCCL otherwise)
                    if a.zero:
                        a.heap.all_reduce_(r.grads)
                    else:
                        dist.all_reduce(r.grads, group=a.dp_group)
                if R > 1 and r.replicated:
                    dist.all_reduce(r.grads, group=a.replicate_group)
                ER = a.expert_rep_world if not r.replicated else 1
                if ER > 1:   # copies of this expert shard on other data-parallel ranks
                    dist.all_reduce(r.grads, group=a.expert_replica_group)
                if r.sp_group is not None:
                    dist.all_reduce(r.grads, group=r.sp_group)
                _lib.call("sumsq", r.grads, _lib.LL(r.grads.numel()), part)
                # scale of these gradients relative to the final ones: inv; replicated ones (and the copies of an
                # expert shard) are counted once per holder in the global sum below
                s = inv * inv / (N if (N > 1 and r.replicated) else ER)
                part.mul_(s)
        tp_idx = [i for i, r in enumerate(a.regions.values()) if r.tp_group is not None]
        if tp_idx:
            # squared norms of tensor-parallel shards add up over the TP group; everything else is identical on the
            # TP peers and counts once: [rest, shards] -> data-parallel sum of both -> TP sum of the second
            P = self._partial.view(len(a.regions), stride)
            self._tot2[1] = P[tp_idx].sum()
            self._tot2[0] = P.sum() - self._tot2[1]
            if N > 1:
                if a.zero:
                    a.heap.all_reduce_(self._tot2)
                else:
                    dist.all_reduce(self._tot2, group=a.dp_group)
            dist.all_reduce(self._tot2[1:], group=next(r.tp_group for r in a.regions.values() if r.tp_group is not None))
            self._partial.zero_()
            self._partial[:1].copy_(self._tot2.sum(dim=0, keepdim=True))
        elif N > 1:
            torch.sum(self._partial, dim=0, keepdim=True, out=self._tot)
            if a.zero:
                a.heap.all_reduce_(self._tot)
            else:
                dist.all_reduce(self._tot, group=a.dp_group)
            self._partial.zero_()
            self._partial[:1].copy_(self._tot)
        if self.norm_groups:
            torch.sum(self._partial, dim=0, keepdim=True, out=self._tot)
            for g in self.norm_groups:
                dist.all_reduce(self._tot, group=g)
            self._partial.zero_()
            self._partial[:1].copy_(self._tot / self.norm_copies)
        _lib.call("clip_coef", self._partial, self._partial.numel(), extra,
                  float(self.max_grad_norm or 0.0), self._coef)
        self.last_grad_norm = self._coef[1]
        torch.mul(self._coef[:1], inv, out=self._coef_local)  # coefficient for gradients not yet divided
        main = torch.cuda.current_stream() if self._cuda else None
        two_stream = a.zero and any(not (r.replicated and r.dtype == torch.bfloat16) and r.weights.numel() > (1 << 24)
                                    for r in a.regions.values())
        if two_stream:
            # the sharded update ends in peer stores of the new weights (NVLink-bound), the update of the local (expert)
            # regions is HBM-bound: run the first on a side stream under the second
            self._side2.wait_stream(main)
        for r in a.regions.values():
            wdr = wd if r.decay else 0.0
            zero_region = a.zero and r.replicated and r.dtype == torch.bfloat16
            with torch.cuda.stream(self._side2 if (two_stream and zero_region) else main):
                self._update_region(r, lr, b1, b2, eps, wdr, N)
        if two_stream:
            main.wait_stream(self._side2)
        if a.zero:
            a.heap.barrier()  # all ranks' weight stores have landed before the next forward reads them
            a.heap.end_step()
        for hook in self.post_step_hooks:
            hook()
        return None

    def _update_region(self, r, lr, b1, b2, eps, wdr, N):
        a = self.arena
        if True:
            if a.zero and r.replicated and r.dtype == torch.bfloat16 and r.mc_weights:
                _lib.check(_lib.lib().np_zero_adamw_bcast_mc(
                    C.c_void_p(r.master.data_ptr()), C.c_void_p(r.gshard.data_ptr()), C.c_void_p(r.m.data_ptr()),
                    C.c_void_p(r.v.data_ptr()), C.c_void_p(r.mc_weights), C.c_longlong(r.lo), C.c_longlong(r.cnt),
                    C.c_float(lr), C.c_float(b1), C.c_float(b2), C.c_float(eps), C.c_float(wdr), self.step_count,
                    C.c_void_p(self._coef.data_ptr()), C.c_void_p(self._hyper.data_ptr()),
                    C.c_void_p(_lib.stream())), "zero_adamw_bcast_mc")
            elif a.zero and r.replicated and r.dtype == torch.bfloat16:
                ptrs = a.heap.host_ptr_array(r.weights)
                _lib.check(_lib.lib().np_zero_adamw_bcast(
                    C.c_void_p(r.master.data_ptr()), C.c_void_p(r.gshard.data_ptr()), C.c_void_p(r.m.data_ptr()),
                    C.c_void_p(r.v.data_ptr()), ptrs, N, C.c_longlong(r.lo), C.c_longlong(r.cnt), C.c_float(lr),
                    C.c_float(b1), C.c_float(b2), C.c_float(eps), C.c_float(wdr), self.step_count,
                    C.c_void_p(self._coef.data_ptr()), C.c_void_p(self._hyper.data_ptr()),
                    C.c_longlong(r.slice if r.bucket else 0), C.c_longlong(r.bucket),
                    C.c_void_p(_lib.stream())), "zero_adamw_bcast")
            elif r.dtype == torch.float32:
                _lib.call("adamw", r.weights, r.grads, r.m, r.v, None, _lib.LL(r.weights.numel()), float(lr),
                          float(b1), float(b2), float(eps), float(wdr), self.step_count, self._coef_local, self._hyper)
            else:
                _lib.call("adamw", r.master, r.grads, r.m, r.v, r.weights, _lib.LL(r.weights.numel()), float(lr),
                          float(b1), float(b2), float(eps), float(wdr), self.step_count, self._coef_local, self._hyper)

    def _step_reference(self, lr, b1, b2, eps, wd):
        """CPU path: same math with torch ops (also the oracle of the kernels)."""
        a = self.arena
        N = a.world
        inv = 1.0 / (self.grad_divisor * (N if N > 1 else 1) * a.rep_world)
        sq = torch.zeros(2, dtype=torch.float32, device=a.device)   # [whole parameters, tensor-parallel shards]
        tpg = None
        for r in a.regions.values():
            if N > 1 and r.replicated:
                dist.all_reduce(r.grads, group=a.dp_group)
            if a.rep_world > 1 and r.replicated:
                dist.all_reduce(r.grads, group=a.replicate_group)
            ER = a.expert_rep_world if not r.replicated else 1
            if ER > 1:
                dist.all_reduce(r.grads, group=a.expert_replica_group)
            if r.sp_group is not None:
                dist.all_reduce(r.grads, group=r.sp_group)
            s = (r.grads.float() * inv).pow(2).sum()
            sq[1 if r.tp_group is not None else 0] += s / (N if (N > 1 and r.replicated) else ER)
            tpg = r.tp_group if r.tp_group is not None else tpg
        if N > 1:
            dist.all_reduce(sq, group=a.dp_group)
        if tpg is not None:
            dist.all_reduce(sq[1:], group=tpg)
        tot = sq.sum()
        for g in self.norm_groups:
            dist.all_reduce(tot, group=g)
        norm = (tot / self.norm_copies).sqrt()
        for hook in self.post_step_hooks:
            hook()
        coef = torch.clamp(self.max_grad_norm / (norm + 1e-6), max=1.0) if self.max_grad_norm else torch.ones(())
        self.last_grad_norm = norm
        t = self.step_count
        for r in a.regions.values():
            gsc = r.grads * (inv * coef)
            tgt = r.master if r.master is not None else r.weights
            r.m.mul_(b1).add_(gsc, alpha=1 - b1)
            r.v.mul_(b2).addcmul_(gsc, gsc, value=1 - b2)
            tgt.mul_(1 - lr * (wd if r.decay else 0.0))
            tgt.addcdiv_(r.m / (1 - b1 ** t), (r.v / (1 - b2 ** t)).sqrt() + eps, value=-lr)
            if r.master is not None:
                r.weights.copy_(r.master)
        return None

    # ------------------------------------------------------------------ (de)serialisation
    def state_dict(self):
        a = self.arena
        return {"step": self.step_count, "param_groups": [{k: v for k, v in g.items() if k != "params"}
                                                          for g in self.param_groups],
                "regions": {k: {"master": r.master, "m": r.m, "v": r.v, "lo": r.lo, "cnt": r.cnt, "bucket": r.bucket}
                            for k, r in a.regions.items()},
                # how the state above is cut, so that a run on another number of ranks can put it together again
                "layout": {"world": a.world, "rank": a.rank,
                           "regions": {k: {"numel": r.numel, "total": r.weights.numel(), "replicated": r.replicated,
                                           "sharded": bool(r.cnt != r.weights.numel())}
                                       for k, r in a.regions.items()}}}

    def load_state_dict_resharded(self, by_rank: List[dict]):
        """Restore from the optimizer states of *all* ranks of a run with another data-parallel size (``by_rank[i]``:
        what rank i saved). Sharded regions are put together from every rank's part, cut to the parameters' length
        (the padding depends on the old world size) and cut again the way this arena shards them. Expert-sharded
        regions hold other experts on every rank: they can only be taken over when the expert placement is unchanged,
        which a different world size rules out, so that case raises instead of loading the wrong experts."""
        first = by_rank[0]
        old = first.get("layout")
        if old is None:
            raise ValueError("this checkpoint predates the layout record needed for re-sharding")
        assert len(by_rank) == old["world"], "need the optimizer state of every rank of the saved run"
        self.step_count = first["step"]
        for g, s in zip(self.param_groups, first["param_groups"]):
            g.update(s)
        a = self.arena
        for k, r in a.regions.items():
            lay = old["regions"].get(k)
            if lay is None:
                raise KeyError(f"region {k} is not in the checkpoint")
            if not r.replicated and a.world != old["world"]:
                raise ValueError(f"region {k} is expert-sharded: the expert placement of a {old['world']}-rank run "
                                 f"cannot be mapped onto {a.world} ranks")
            total_new = r.weights.numel()
            for name in ("master", "m", "v"):
                cur = getattr(r, name)
                if cur is None:
                    continue
                parts = [sd["regions"][k][name] for sd in by_rank]
                if any(p_ is None for p_ in parts):
                    continue
                if lay["sharded"]:
                    full = assemble_shards([p_.reshape(-1) for p_ in parts], first["regions"][k]["bucket"])
                else:
                    full = parts[min(a.rank, len(parts) - 1)].reshape(-1) if not r.replicated else parts[0].reshape(-1)
                full = full[:lay["numel"]]
                flat = torch.zeros(total_new, dtype=cur.dtype)
                flat[:full.numel()] = full.to(cur.dtype)
                piece = owned_slice(flat, a.world, a.rank, r.bucket) if cur.numel() != total_new else flat
                cur.copy_(piece.to(cur.device))

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for g, s in zip(self.param_groups, sd["param_groups"]):
            g.update(s)
        for k, st in sd["regions"].items():
            r = self.arena.regions[k]
            for name in ("master", "m", "v"):
                if st[name] is not None and getattr(r, name) is not None:
                    getattr(r, name).copy_(st[name])
