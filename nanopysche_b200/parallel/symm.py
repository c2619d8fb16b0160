"""Symmetric device memory shared by the ranks of one node.

Each rank allocates one arena (``cudaMalloc``), exports its CUDA IPC handle, and opens every other
rank's; tensors carved out of the arena have the same offset on every rank, so a kernel addresses
"buffer X on rank r" as ``peer_base[r] + offset``. ``torch.distributed`` is used only to exchange
the 64-byte handles. A single-rank heap needs no IPC and uses ordinary torch memory.

Kernels signal through epoch flags (monotone counters) that live in the arena; every wait on a
flag is bounded and reports through the library's status word instead of hanging.

The reference has no counterpart: its collectives are NCCL calls (model/moe.py:396-497,
model/tp_utils.py:38); this heap is what lets dispatch, combine, reduce-scatter and all-gather run
inside the compute kernels.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _lib


def available() -> bool:
    return torch.cuda.is_available()


class _RawCuda:
    """Array-interface view of raw device memory so torch can wrap it without a copy."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class SymmetricHeap:
    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        # group=None means "this rank alone" (pass dist.group.WORLD explicitly for all ranks)
        self.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        self.rank = dist.get_rank(group) if self.world > 1 else 0
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = int(math.ceil(nbytes / 4096) * 4096)
        self._offset = 0
        self._ipc = self.world > 1
        if not self._ipc:
            self._base_tensor = torch.zeros(self.nbytes, dtype=torch.uint8, device=self.device)
            self.local_ptr = self._base_tensor.data_ptr()
            self.peer_ptrs = [self.local_ptr]
        else:
            lib = _lib.lib()
            ptr = C.c_void_p()
            handle = (C.c_ubyte * 64)()
            _lib.check(lib.np_symm_alloc(C.c_ulonglong(self.nbytes), C.byref(ptr), handle), "symm_alloc")
            self.local_ptr = ptr.value
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle), group=group)
            self.peer_ptrs = []
            for r, h in enumerate(handles):
                if r == self.rank:
                    self.peer_ptrs.append(self.local_ptr)
                    continue
                p = C.c_void_p()
                buf = (C.c_ubyte * 64).from_buffer_copy(h)
                _lib.check(lib.np_symm_open(buf, C.byref(p)), "symm_open")
                self.peer_ptrs.append(p.value)
            self._base_tensor = torch.as_tensor(_RawCuda(self.local_ptr, self.nbytes), device=self.device)
        # Epochs are ``*epoch_base + offset``: the offset is a host integer that restarts every step, the
        # base lives on the device and is advanced by ``end_step()`` with an ordinary stream-ordered add,
        # so a captured CUDA graph of one step replays with fresh, still monotone epochs.
        self.epoch_base = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._epoch_off = 0
        self._barrier_flags = self.alloc((self.world,), torch.int32)
        self._ar_flags = self.alloc((self.world,), torch.int32)
        self._ar_ctr = torch.zeros(2, dtype=torch.int32, device=self.device)
        self._ar_half = 0
        self._ar_staging = None

    # -- allocation --------------------------------------------------------------------------------
    def alloc(self, shape, dtype: torch.dtype, align: int = 256) -> torch.Tensor:
        """Carve a zero-initialised tensor out of the arena (same offset on every rank when all ranks
        allocate in the same order)."""
        n = int(math.prod(shape)) * torch.empty((), dtype=dtype).element_size()
        off = (self._offset + align - 1) // align * align
        if off + n > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted: need {off + n} of {self.nbytes} bytes")
        self._offset = off + n
        t = self._base_tensor[off:off + n].view(dtype).view(*shape)
        t._symm_offset = off
        return t

    def offset_of(self, t: torch.Tensor) -> int:
        return t.data_ptr() - self.local_ptr

    def peer_ptr(self, t: torch.Tensor, rank: int) -> int:
        return self.peer_ptrs[rank] + self.offset_of(t)

    def ptr_array(self, t: torch.Tensor) -> torch.Tensor:
        """Device int64 tensor ``[world]``: address of ``t`` on every rank (a ``void* const*`` for kernels)."""
        return torch.tensor([self.peer_ptr(t, r) for r in range(self.world)], dtype=torch.int64,
                            device=self.device)

    def host_ptr_array(self, t: torch.Tensor):
        arr = (C.c_void_p * self.world)(*[self.peer_ptr(t, r) for r in range(self.world)])
        return arr

    # -- synchronisation -----------------------------------------------------------------------------
    def next_epoch(self) -> int:
        self._epoch_off += 1
        return self._epoch_off

    def end_step(self):
        """Fold this step's epoch offsets into the device-side base (call once per optimizer step)."""
        if self._epoch_off:
            self.epoch_base.add_(self._epoch_off)
            self._epoch_off = 0

    def barrier(self, limit_ns: int = 0):
        """Device-side barrier on the current stream (no host synchronisation)."""
        if self.world <= 1:
            return
        arr = self.host_ptr_array(self._barrier_flags)
        _lib.check(_lib.lib().np_symm_barrier(arr, self.rank, self.world, self.next_epoch(),
                                              C.c_void_p(self.epoch_base.data_ptr()), C.c_ulonglong(limit_ns),
                                              C.c_void_p(_lib.stream())), "symm_barrier")

    def reserve_allreduce(self, max_count: int):
        """Allocate the staging area of ``all_reduce_`` (every rank, same order as other allocations)."""
        self._ar_half = self.world * max_count
        self._ar_staging = self.alloc((2 * self._ar_half,), torch.float32)

    def all_reduce_(self, t: torch.Tensor, scale: float = 1.0, limit_ns: int = 0) -> torch.Tensor:
        """In-place sum of a (small) fp32 tensor over the ranks through peer stores; no NCCL involved."""
        if self.world <= 1:
            if scale != 1.0:
                t.mul_(scale)
            return t
        assert t.dtype == torch.float32 and t.is_contiguous() and self._ar_staging is not None
        assert self.world * t.numel() <= self._ar_half, "reserve_allreduce() was sized too small"
        st, fl = self.host_ptr_array(self._ar_staging), self.host_ptr_array(self._ar_flags)
        _lib.check(_lib.lib().np_symm_allreduce(
            C.c_void_p(t.data_ptr()), C.c_void_p(t.data_ptr()), st, fl, C.c_void_p(self._ar_ctr.data_ptr()),
            C.c_longlong(self._ar_half), C.c_longlong(t.numel()), self.rank, self.world, self.next_epoch(),
            C.c_void_p(self.epoch_base.data_ptr()), C.c_float(scale), C.c_ulonglong(limit_ns),
            C.c_void_p(_lib.stream())), "symm_allreduce")
        return t

    def close(self, collective: bool = True):
        """Unmap the peers' memory and free this rank's. ``collective=True`` brackets the unmapping with two barriers
        so that no rank frees memory a peer still has mapped and in use; after a peer has left the job
        (``PeerLeftError``, ``CommTimeoutError``) pass ``collective=False``: a barrier would wait for the departed
        rank, and nothing of this heap is launched any more."""
        if self._ipc:
            lib = _lib.lib()
            torch.cuda.synchronize()
            if collective and dist.is_initialized():
                dist.barrier(group=self.group)
            for r, p in enumerate(self.peer_ptrs):
                if r != self.rank:
                    lib.np_symm_close(C.c_void_p(p))
            if collective and dist.is_initialized():
                dist.barrier(group=self.group)
            lib.np_symm_free(C.c_void_p(self.local_ptr))
            self._ipc = False


def nvls_alloc(numel: int, dtype: torch.dtype, group, device):
    """A flat tensor in symmetric memory that is also bound to an NVLink multicast object (NVLS), for kernels that
    use ``multimem.ld_reduce`` / ``multimem.st`` on it. The allocation, the handle exchange between the ranks and the
    multicast binding are PyTorch's (``torch.distributed._symmetric_memory``); the kernels only need the multicast
    address. Returns ``(tensor, multicast_address, handle)`` or ``None`` when not switched on (``NPB200_NVLS=1``) or
    when any rank of the group has no multicast mapping. Collective over ``group``.

    Off by default: measured on 8 B200 the data-parallel step takes the same time either way (a reduce-scatter
    still sends 7/8 of every rank's gradients out, an all-gather still receives 7/8 of the weights; the switch only
    relieves the other direction), and memory bound to a multicast object makes the death of one rank a fault on
    its peers."""
    import os

    if os.environ.get("NPB200_NVLS", "0") != "1" or group is None:
        return None
    t, mc, hdl = None, 0, None
    try:
        import torch.distributed._symmetric_memory as sm

        t = sm.empty(int(numel), dtype=dtype, device=device)
        hdl = sm.rendezvous(t, group)
        mc = int(getattr(hdl, "multicast_ptr", 0) or 0)
    except Exception:  # noqa: BLE001 - any failure means "no NVLS here"
        mc = 0
    flag = torch.tensor([1 if mc else 0], device=device, dtype=torch.int32)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    if int(flag.item()) == 0:
        return None
    return t, mc, hdl
