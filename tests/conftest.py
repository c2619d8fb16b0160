"""Test configuration: the ``gpu`` marker, repo root on ``sys.path``, and a helper that runs a
function on N gloo ranks (CPU) or N NCCL ranks (GPU) as child processes."""
import os
import socket
import sys
import traceback

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for it in items:
        if "gpu" in it.keywords:
            it.add_marker(skip)


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, backend, fn, args, q):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank), GLOO_SOCKET_IFNAME="lo", NCCL_NVLS_ENABLE="0")
    try:
        if backend == "nccl":
            torch.cuda.set_device(rank)
        dist.init_process_group(backend, rank=rank, world_size=world)
        res = fn(rank, world, *args)
        q.put((rank, "ok", res))
    except BaseException as e:  # noqa: BLE001
        q.put((rank, "err", f"{type(e).__name__}: {e}\n{traceback.format_exc()}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001
            pass


class _RendezvousTrouble(Exception):
    """A rank failed while the process group was being set up or torn down (a port taken between choosing and
    binding it, a connection reset by a process that is still exiting), not in the code under test."""


def run_distributed(fn, world: int, *args, backend: str = "gloo", timeout: float = 240.0):
    """Run ``fn(rank, world, *args)`` on ``world`` ranks; returns the per-rank results, raises on any
    failure. ``fn`` must be a module-level function (spawned processes import it by name). A failure of the
    rendezvous itself (gloo, on the CPU box) is retried once on a fresh port; a failure in ``fn`` never is."""
    if backend != "gloo":
        return _run_distributed_once(fn, world, args, backend, timeout)
    try:
        return _run_distributed_once(fn, world, args, backend, timeout)
    except _RendezvousTrouble:
        return _run_distributed_once(fn, world, args, backend, timeout)


_RENDEZVOUS_MARKS = ("Address already in use", "Connection reset by peer", "Connection refused",
                     "Connection closed by peer", "Broken pipe", "connectFullMesh", "Socket Timeout",
                     "store-based barrier")


def _run_distributed_once(fn, world, args, backend, timeout):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, backend, fn, args, q)) for r in range(world)]
    for p in procs:
        p.start()
    out = {}
    try:
        for _ in range(world):
            rank, status, payload = q.get(timeout=timeout)
            if status != "ok":
                if "AssertionError" not in payload and any(m in payload for m in _RENDEZVOUS_MARKS):
                    raise _RendezvousTrouble(payload)
                raise AssertionError(f"rank {rank} failed:\n{payload}")
            out[rank] = payload
    finally:
        for p in procs:
            p.join(timeout=10)
            if p.is_alive():
                p.kill()
    return [out[r] for r in range(world)]
