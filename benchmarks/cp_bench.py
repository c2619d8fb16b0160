"""Context-parallel attention benchmark: ``torchrun --nproc-per-node N -m benchmarks.cp_bench``.

Times forward + backward of attention over a sequence sharded over the ``N`` ranks (zig-zag layout) for

* ``ring_fused``    - one flash kernel per rank that pulls the peers' K/V (and Q/dO for dK/dV) tiles over NVLink,
* ``ulysses_fused`` - Ulysses with the head/sequence exchange inside the kernels' loads and stores,
* ``ulysses_nccl``  - four NCCL all-to-alls around the single-GPU flash kernels (the reference's structure,
                      distributed/context_parallel.py:334-375, with a flash kernel instead of dense softmax),

with CUDA events on every rank (max over ranks), and prints one JSON line per variant with the achieved
TFLOP/s per GPU, the bytes each rank moves over NVLink and the fraction of the roofline (slower of FLOPs at the
measured GEMM peak and bytes at 770 GB/s per direction).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=32768, help="total sequence length")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--variants", default="ring_fused,ulysses_fused,ulysses_nccl")
    a = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    rank, world = dist.get_rank(), dist.get_world_size()
    from nanopysche_b200.ops import _lib
    from benchmarks.microbench import peaks
    from nanopysche_b200.parallel.context_parallel import RingAttention

    dev = torch.device("cuda", local)
    S = a.seq // world
    torch.manual_seed(rank)
    q = torch.randn(a.batch, S, a.heads, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(a.batch, S, a.kv_heads, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(a.batch, S, a.kv_heads, 128, device=dev, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn_like(q)
    _, tf, src = peaks()
    flops = 3.5 * 4.0 * a.batch * a.heads * a.seq * a.seq * 128 * 0.5 / world       # fwd + bwd, causal, per rank
    qb, kb = q.numel() * 2, k.numel() * 2
    nv = {"ring_fused": (world - 1) * (2 * kb) + (world - 1) * (2 * kb + 2 * qb),       # K,V fwd; K,V,Q,dO bwd
          "ulysses_fused": (world - 1) / world * (2 * qb + 2 * kb) + (world - 1) / world * (3 * qb + 4 * kb + 2 * qb),
          "ulysses_nccl": (world - 1) / world * 2 * (2 * qb + 2 * kb)}
    mods = {"ring_fused": RingAttention(dist.group.WORLD, use_zigzag=True, fused=True),
            "ulysses_fused": RingAttention(dist.group.WORLD, use_ulysses=True, use_zigzag=True, fused=True),
            "ulysses_nccl": RingAttention(dist.group.WORLD, use_ulysses=True, use_zigzag=True, fused=False)}
    for name in a.variants.split(","):
        mod = mods[name]

        def step():
            q.grad = k.grad = v.grad = None
            mod(q, k, v, causal=True).backward(g)

        for _ in range(2):
            step()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.iters):
            step()
        e1.record()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1) / a.iters], device=dev)
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        ms = ms.item()
        _lib.check_status(name)
        t_roof = max(flops / (tf * 1e12), nv[name] / 770e9) * 1e3
        if rank == 0:
            print(json.dumps({"variant": name, "world": world, "seq": a.seq, "batch": a.batch, "heads": a.heads,
                              "kv_heads": a.kv_heads, "ms_fwd_bwd": ms, "tflops_per_gpu": flops / ms / 1e9,
                              "nvlink_bytes_per_rank": nv[name], "roofline_ms": t_roof,
                              "frac_of_roofline_" + src: t_roof / ms}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
