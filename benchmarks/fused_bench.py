"""Fused compute+collective linears against their NCCL baselines:
``torchrun --nproc-per-node N -m benchmarks.fused_bench [--tokens 4096 --d-model 2048 --ffn 5632]``.

Variants (forward only, CUDA events on every rank, max over ranks, median of ``--iters``):

* ``tp_ag_gemm``  all-gather(x shard) -> GEMM (column-parallel linear, sequence-parallel input)
                  fused: push kernel + tcgen05 GEMM waiting per 128-row block; baseline: NCCL all-gather, then GEMM
* ``tp_gemm_rs``  GEMM -> reduce-scatter (row-parallel linear)
                  fused: GEMM epilogue stores rows into the owner's slots + sum; baseline: GEMM, then NCCL reduce-scatter
* ``fsdp_ag_gemm`` all-gather(weight shard) -> GEMM
                  fused: push kernel + GEMM waiting per weight shard; baseline: NCCL all-gather, then GEMM

Each line reports the time, the fraction of the roofline (slower of FLOPs at the measured GEMM peak and bytes over
NVLink at 770 GB/s per direction) and the baseline's time. The baseline GEMM is this library's kernel too, so the
difference is the overlap.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist


def _time(fn, iters, dev):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4096)
    ap.add_argument("--d-model", type=int, default=2048)
    ap.add_argument("--ffn", type=int, default=5632)
    ap.add_argument("--iters", type=int, default=11)
    a = ap.parse_args(argv)
    local = int(os.environ.get("LOCAL_RANK", 0))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")
    rank, n = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", local)
    from nanopysche_b200.ops import _lib, tp_fused
    from nanopysche_b200.ops.fsdp_fused import FSDPRuntime
    from nanopysche_b200.ops.gemm import gemm
    from benchmarks.microbench import peaks

    _, tf, src = peaks()
    M, D, F = a.tokens, a.d_model, a.ffn
    Fl = F // n
    bf = torch.bfloat16
    torch.manual_seed(rank)
    rt = tp_fused.TPRuntime(dist.group.WORLD, rows=M, max_cols=max(D, Fl))
    x_shard = torch.randn(M // n, D, device=dev, dtype=bf)
    w_col = torch.randn(Fl, D, device=dev, dtype=bf) * 0.02     # column-parallel weight shard
    h = torch.randn(M, Fl, device=dev, dtype=bf)
    w_row = torch.randn(D, Fl, device=dev, dtype=bf) * 0.02     # row-parallel weight shard
    full = torch.empty(M, D, device=dev, dtype=bf)
    out = []

    def report(name, t_fused, t_base, flops, nvbytes):
        roof = max(flops / (tf * 1e12), nvbytes / 770e9) * 1e3
        if rank == 0:
            print(json.dumps({"variant": name, "world": n, "ms_fused": t_fused, "ms_nccl_then_gemm": t_base,
                              "speedup": t_base / t_fused, "roofline_ms": roof,
                              "frac_of_roofline_" + src: roof / t_fused}), flush=True)

    # all-gather -> GEMM
    def ag_fused():
        rt.ag_gemm(x_shard, w_col, b_mn=False)

    def ag_base():
        dist.all_gather_into_tensor(full, x_shard)
        gemm(full, w_col)

    report("tp_ag_gemm", _time(ag_fused, a.iters, dev), _time(ag_base, a.iters, dev), 2.0 * M * D * Fl,
           (n - 1) * x_shard.numel() * 2)

    # GEMM -> reduce-scatter
    y_full = torch.empty(M, D, device=dev, dtype=bf)
    y_shard = torch.empty(M // n, D, device=dev, dtype=bf)

    def rs_base():
        y = gemm(h, w_row)
        dist.reduce_scatter_tensor(y_shard, y)

    report("tp_gemm_rs", _time(lambda: rt.gemm_reduce_scatter(h, w_row, b_mn=False), a.iters, dev),
           _time(rs_base, a.iters, dev), 2.0 * M * Fl * D, (n - 1) * (M // n) * D * 2)
    report("tp_gemm_rs_push_epilogue", _time(lambda: rt.gemm_reduce_scatter_push(h, w_row, b_mn=False), a.iters, dev),
           _time(rs_base, a.iters, dev), 2.0 * M * Fl * D, (n - 1) * (M // n) * D * 2)

    # FSDP: all-gather(weight) -> GEMM
    frt = FSDPRuntime(dist.group.WORLD, max_weight_elems=F * D)
    w_shard = torch.randn(F // n, D, device=dev, dtype=bf) * 0.02
    x = torch.randn(M, D, device=dev, dtype=bf)
    w_full = torch.empty(F, D, device=dev, dtype=bf)

    def fsdp_fused():
        frt.ag_gemm(x, w_shard)

    def fsdp_base():
        dist.all_gather_into_tensor(w_full, w_shard)
        gemm(x, w_full)

    report("fsdp_ag_gemm", _time(fsdp_fused, a.iters, dev), _time(fsdp_base, a.iters, dev), 2.0 * M * D * F,
           (n - 1) * w_shard.numel() * 2)
    torch.cuda.synchronize()
    _lib.check_status("fused_bench")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
