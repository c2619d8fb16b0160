"""Bucketed data-parallel gradient all-reduce that overlaps with the backward pass.

The reference names DDP only as an enum value (distributed/fsdp.py:35) and has no code for it. This is the plain
(un-sharded) data-parallel path of this framework for models that do not use the parameter arena: parameters are
grouped into buckets in reverse registration order (roughly the order their gradients become ready); a
post-accumulate hook copies each gradient into its bucket's flat buffer, and the bucket's all-reduce is launched
asynchronously as soon as its last gradient has arrived, so the collective of the later layers runs under the
backward pass of the earlier ones. ``finish()`` waits, averages and writes the results back into ``p.grad``.

Only the ranks of ``group`` take part: pass the *replica* group (dp x ep x cp), never the world when tensor or
pipeline parallelism is on, because TP / PP peers hold different shards.
"""
from __future__ import annotations

from typing import Iterable, List, Optional

import torch
import torch.distributed as dist


class _Bucket:
    def __init__(self, params: List[torch.nn.Parameter]):
        self.params = params
        self.offsets, n = [], 0
        for p in params:
            self.offsets.append(n)
            n += p.numel()
        self.numel = n
        self.flat: Optional[torch.Tensor] = None
        self.pending = len(params)
        self.seen = set()
        self.work = None


class BucketedGradReducer:
    def __init__(self, params: Iterable[torch.nn.Parameter], group=None, bucket_bytes: int = 64 << 20,
                 average: bool = True, divisor: Optional[float] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.average = average
        # what the summed gradients are divided by: the group size, or less when some ranks of the group hold shares
        # of one sample's gradient that must add up (context parallelism)
        self.divisor = float(divisor) if divisor else float(self.world)
        self.enabled = True          # the trainer switches this off for all but the last micro-batch of a step
        self.buckets: List[_Bucket] = []
        self._of = {}
        cur, cur_bytes, cur_key = [], 0, None
        for p in reversed([p for p in params if p.requires_grad]):
            key = (p.dtype, p.device)
            nbytes = p.numel() * p.element_size()
            if cur and (key != cur_key or cur_bytes + nbytes > bucket_bytes):
                self.buckets.append(_Bucket(cur))
                cur, cur_bytes = [], 0
            cur.append(p)
            cur_bytes += nbytes
            cur_key = key
        if cur:
            self.buckets.append(_Bucket(cur))
        self._handles = []
        for b in self.buckets:
            for p, off in zip(b.params, b.offsets):
                self._of[id(p)] = (b, off)
                self._handles.append(p.register_post_accumulate_grad_hook(self._hook))

    def _hook(self, p):
        if not self.enabled or self.world <= 1 or p.grad is None:
            return
        b, off = self._of[id(p)]
        if b.flat is None:
            b.flat = torch.zeros(b.numel, dtype=p.grad.dtype, device=p.grad.device)
        b.flat[off:off + p.numel()].copy_(p.grad.reshape(-1))
        b.seen.add(id(p))
        b.pending -= 1
        if b.pending == 0:
            b.work = dist.all_reduce(b.flat, group=self.group, async_op=True)

    def finish(self):
        """Wait for every bucket (launching those whose parameters did not all receive a gradient), average and
        copy back. Call once per optimizer step, after the last backward."""
        if self.world <= 1:
            return
        for b in self.buckets:
            if b.work is None:
                # not every parameter came through the hook: it had no gradient this step, or its gradient was set
                # outside autograd (weight gradients deferred by a zero-bubble schedule); every rank sends the bucket
                ref = next((p for p in b.params if p.grad is not None), None)
                if b.flat is None:
                    b.flat = torch.zeros(b.numel, dtype=ref.grad.dtype if ref is not None else b.params[0].dtype,
                                         device=b.params[0].device)
                for p, off in zip(b.params, b.offsets):
                    if id(p) in b.seen:
                        continue
                    if p.grad is None:
                        b.flat[off:off + p.numel()].zero_()
                    else:
                        b.flat[off:off + p.numel()].copy_(p.grad.reshape(-1))
                b.work = dist.all_reduce(b.flat, group=self.group, async_op=True)
        for b in self.buckets:
            if b.work is not None:
                b.work.wait()
                if self.average:
                    b.flat.div_(self.divisor)
                for p, off in zip(b.params, b.offsets):
                    if p.grad is not None:
                        p.grad.copy_(b.flat[off:off + p.numel()].view_as(p.grad))
            b.work, b.pending = None, len(b.params)
            b.seen.clear()

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []
