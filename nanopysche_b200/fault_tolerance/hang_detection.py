"""Hang detection (reference: fault_tolerance/hang_detection.py:38-219).

``HangDetector`` is a watchdog thread fed by ``heartbeat()`` once per step; when the heartbeat is
older than ``timeout`` it calls ``on_hang`` and aborts the process group. ``HeartbeatCoordinator``
publishes every rank's step counter through a host-side key-value store (the job's ``TCPStore`` or an
in-process dict) - never through a GPU collective from a side thread, and every rank takes part
(in the reference only rank 0 enters an all-gather, which would itself hang). A rank whose counter
has not moved for ``hang_timeout`` seconds is reported through ``on_stall``.
"""
from __future__ import annotations

import threading
import time
from typing import Callable, Dict, List, Optional

import torch.distributed as dist


class CommTimeoutError(RuntimeError):
    """A bounded device-side or collective wait ran out."""


class PeerLeftError(CommTimeoutError):
    """A peer announced that it leaves the job (preemption, planned shrink): raised on the remaining ranks before they
    launch the step the peer will no longer take part in."""


class HangDetector:
    def __init__(self, timeout: float = 300.0, check_interval: float = 10.0, on_hang: Optional[Callable] = None,
                 abort_on_hang: bool = True):
        self.timeout, self.check_interval, self.on_hang, self.abort_on_hang = timeout, check_interval, on_hang, \
            abort_on_hang
        self._last = time.monotonic()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.hang_detected = False

    def start(self):
        self._last = time.monotonic()
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True, name="hang-detector")
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.check_interval + 1)
            self._thread = None

    def heartbeat(self):
        self._last = time.monotonic()

    def _run(self):
        while not self._stop.wait(self.check_interval):
            if time.monotonic() - self._last > self.timeout:
                self.hang_detected = True
                if self.on_hang is not None:
                    try:
                        self.on_hang()
                    except Exception:  # noqa: BLE001
                        pass
                if self.abort_on_hang and dist.is_available() and dist.is_initialized():
                    try:
                        dist.destroy_process_group()
                    except Exception:  # noqa: BLE001
                        pass
                return

    @staticmethod
    def check_collective_timeout(collective_fn: Callable, timeout: float = 60.0, *, raise_on_timeout: bool = False) -> bool:
        """Run ``collective_fn()``; returns True when it ended in what looks like a collective timeout, False when it
        completed (reference: fault_tolerance/hang_detection.py:113-129); any other exception propagates. With
        ``raise_on_timeout`` the timeout is raised as ``CommTimeoutError`` instead. ``timeout`` is accepted for the
        reference's signature: how long a collective may take is a property of its process group
        (``init_process_group(timeout=...)``), not of this call."""
        try:
            collective_fn()
            return False
        except Exception as e:  # noqa: BLE001
            if "timeout" in str(e).lower() or "timed out" in str(e).lower():
                if raise_on_timeout:
                    raise CommTimeoutError(str(e)) from e
                return True
            raise


class _DictStore:
    def __init__(self):
        self._d: Dict[str, bytes] = {}
        self._lock = threading.Lock()

    def set(self, k, v):
        with self._lock:
            self._d[k] = v if isinstance(v, bytes) else str(v).encode()

    def get(self, k):
        with self._lock:
            return self._d[k]

    def check(self, keys):
        with self._lock:
            return all(k in self._d for k in keys)


class HeartbeatCoordinator:
    def __init__(self, check_interval: float = 30.0, hang_timeout: float = 120.0, group=None, store=None,
                 rank: Optional[int] = None, world_size: Optional[int] = None,
                 on_stall: Optional[Callable[[List[int]], None]] = None, prefix: str = "hb"):
        init = dist.is_available() and dist.is_initialized()
        self.rank = rank if rank is not None else (dist.get_rank(group) if init else 0)
        self.world_size = world_size if world_size is not None else (dist.get_world_size(group) if init else 1)
        if store is None:
            store = None
            if init:
                try:
                    store = dist.distributed_c10d._get_default_store()
                except Exception:  # noqa: BLE001
                    store = None
            store = store or _DictStore()
        self.store, self.prefix = store, prefix
        self.check_interval, self.hang_timeout, self.on_stall = check_interval, hang_timeout, on_stall
        self._step = 0
        self._seen: Dict[int, tuple] = {}
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self.stalled_ranks: List[int] = []
        self.store.set(f"{self.prefix}/{self.rank}", str(0))

    def heartbeat(self, step: Optional[int] = None):
        self._step = self._step + 1 if step is None else step
        self.store.set(f"{self.prefix}/{self.rank}", str(self._step))

    # -- planned departure ----------------------------------------------------------------------------------------
    # A rank leaves only between steps, with none of its kernels or collectives in flight, and says so one step ahead:
    # it writes "I take part up to step k" into the store *before* it enters step k. Step k contains a collective that
    # every rank takes part in, so by the time a peer has finished step k the note is visible to it; every remaining
    # rank therefore finds it at the top of step k + 1, before launching anything that would wait for the departed
    # rank, and all of them stop at the same step.
    def announce_departure(self, last_step: int) -> None:
        self.store.set(f"{self.prefix}/left/{self.rank}", str(int(last_step)))

    def departed(self, step: int) -> List[int]:
        """Ranks whose announced last step is below ``step`` (the step about to start)."""
        gone = []
        for r in range(self.world_size):
            if r == self.rank:
                continue
            key = f"{self.prefix}/left/{r}"
            try:
                if hasattr(self.store, "check") and not self.store.check([key]):
                    continue
                if int(self.store.get(key).decode()) < step:
                    gone.append(r)
            except Exception:  # noqa: BLE001
                continue
        return gone

    def start(self):
        if self.rank != 0:
            return
        self._stop.clear()
        self._thread = threading.Thread(target=self._run, daemon=True, name="heartbeat")
        self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=self.check_interval + 1)
            self._thread = None

    def sync_heartbeats(self) -> dict:
        """One monitoring pass: every rank's step counter as ``{rank: counter}`` (-1: never reported), as the reference
        returns it (fault_tolerance/hang_detection.py:189-196) - read from the store, though, not by an all-gather that
        a hung rank would block. The ranks whose counter has not moved for ``hang_timeout`` are left in
        ``stalled_ranks``."""
        now = time.monotonic()
        stalled, counters = [], {}
        for r in range(self.world_size):
            key = f"{self.prefix}/{r}"
            try:
                if hasattr(self.store, "check") and not self.store.check([key]):
                    val = -1
                else:
                    val = int(self.store.get(key).decode())
            except Exception:  # noqa: BLE001
                val = -1
            counters[r] = val
            prev = self._seen.get(r)
            if prev is None or prev[0] != val:
                self._seen[r] = (val, now)
            elif now - prev[1] >= self.hang_timeout:
                stalled.append(r)
        self.stalled_ranks = stalled
        return counters

    def _run(self):
        while not self._stop.wait(self.check_interval):
            self.sync_heartbeats()
            stalled = self.stalled_ranks
            if stalled:
                if self.on_stall is not None:
                    self.on_stall(stalled)
                return
