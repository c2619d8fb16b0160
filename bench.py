"""Headline benchmark: training tokens/s of the 1B MoE decoder with expert parallelism over all GPUs.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per rank by torchrun)
    python bench.py --impl reference ...                     the unmodified reference from baseline/_ref

Config (per GPU batch 2 x seq 2048, weak scaling): 16 layers, d_model 2048, 16 query / 8 KV heads of
dim 128, every FFN replaced by 8 SwiGLU experts (hidden 2816), top-2 softmax routing, capacity factor
1.25, vocab 32000, RoPE base 10000, random-init N(0, 0.02) weights, uniform random tokens, bf16
compute with fp32 master weights, EP = N. One step = forward + backward + gradient clipping + AdamW.

Timing: W untimed steps, then exactly K steps between CUDA events with a barrier + synchronize on
both sides, max over ranks; the end-to-end figure repeats the K steps with a pinned-host -> device
copy of the tokens and a device -> host read of the loss inside every step. GPU clocks and throttle
reasons are sampled with nvidia-smi during the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
CFG = dict(n_layers=16, d_model=2048, n_heads=16, n_kv_heads=8, ffn_hidden=5632, moe_hidden=2816, num_experts=8,
           top_k=2, capacity_factor=1.25, vocab=32000, batch_per_gpu=2, seq_len=2048, rope_base=10000.0)
METRIC = "tokens/s (device-timed, max over ranks) 1B MoE EP8 at 1/2/4/8 B200 vs ref NCCL"


class ClockSampler:
    """Polls nvidia-smi for this GPU's SM clock and throttle reasons while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.samples, self._stop, self._t = index, [], threading.Event(), None

    def start(self):
        self._t = threading.Thread(target=self._run, daemon=True)
        self._t.start()

    def _run(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-i",
                                      str(self.index)], capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.samples.append([f.strip() for f in out.split(",")])
            except Exception:  # noqa: BLE001
                pass
            self._stop.wait(0.2)

    def stop(self) -> dict:
        self._stop.set()
        if self._t is not None:
            self._t.join(timeout=6)
        sm = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        mx = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for s in self.samples for n, v in zip(names, s[3:7]) if v.lower().startswith("active")})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(self.samples)}


def setup_dist(n_gpus: int):
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, local, world


def timed(step_fn, steps: int, world: int, dev):
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for i in range(steps):
        step_fn(i)
    e.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    ms = torch.tensor([s.elapsed_time(e)], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms) / steps


def run_ours(args, rank, local, world):
    sys.path.insert(0, ROOT)
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.engine import prepare_training
    from nanopysche_b200.models.moe import ExpertParallelConfig
    from nanopysche_b200.ops import _lib

    dev = torch.device("cuda", local)
    torch.manual_seed(1234 + rank)
    c = CFG
    cfg = TransformerConfig(vocab_size=c["vocab"], d_model=c["d_model"], n_layers=c["n_layers"], n_heads=c["n_heads"],
                            n_kv_heads=c["n_kv_heads"], ffn_hidden=c["ffn_hidden"], rope_base=c["rope_base"],
                            max_seq_len=c["seq_len"], qk_norm=False, use_moe=True, num_experts=c["num_experts"],
                            moe_top_k=c["top_k"], moe_interval=1, moe_offset=0, moe_hidden=c["moe_hidden"],
                            moe_capacity_factor=c["capacity_factor"])
    torch.manual_seed(1234)  # identical replicated weights on every rank
    model = cfg.build(dtype=torch.bfloat16, init_device="cuda")
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    if world > 1:
        model.apply_ep(ExpertParallelConfig(ep_size=world, ep_group=dist.group.WORLD))
        model._needs_grad_sync = True
    T = c["batch_per_gpu"] * c["seq_len"]
    opt, arena = prepare_training(model, tokens_per_rank=T, lr=3e-4, weight_decay=0.1, max_grad_norm=1.0,
                                  dp_group=dist.group.WORLD if world > 1 else None,
                                  ep_group=dist.group.WORLD if world > 1 else None)
    model.train()
    torch.manual_seed(99 + rank)
    n_batches = 4  # a small fixed set of random batches, cycled, so the loss trend is meaningful
    host = [torch.randint(0, c["vocab"], (c["batch_per_gpu"], c["seq_len"])).pin_memory() for _ in range(n_batches)]
    devb = [h.to(dev) for h in host]
    last = {}

    def train_step(ids):
        out = model(ids, labels=ids)
        loss = out["loss"] + out["aux_loss"]
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)
        last["loss"] = out["loss"].detach()

    from nanopysche_b200.engine import GraphedTrainStep

    eager_step = train_step
    graphed = None
    if not args.no_graph:
        # the whole step (forward + backward + clip + AdamW) replayed as one CUDA graph
        l0 = _lib.LAUNCHES
        graphed = GraphedTrainStep(model, opt, devb[0], warmup=2).capture()
        per_step = (_lib.LAUNCHES - l0) // 3  # two eager warm-up steps + the captured one

        def train_step(ids):  # noqa: F811
            last["loss"] = graphed.step(ids)

    for i in range(args.warmup):
        train_step(devb[i % n_batches])
    torch.cuda.synchronize()
    _lib.check_status("after warm-up")
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    l0 = _lib.LAUNCHES
    ms = timed(lambda i: train_step(devb[i % n_batches]), args.steps, world, dev)
    launches = (_lib.LAUNCHES - l0) if graphed is None else per_step * args.steps
    clocks = sampler.stop() if rank == 0 else {}
    loss_dev = float(last["loss"].detach())

    def e2e_step(i):
        ids = host[i % n_batches]
        train_step(ids if graphed is not None else ids.to(dev, non_blocking=True))  # graph: copied into its static input
        last["host_loss"] = last["loss"].item()

    ms_e2e = timed(e2e_step, args.steps, world, dev)
    _lib.check_status("after timed region")
    tokens = T * world
    value = tokens / (ms / 1e3)
    res = {
        "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic uniform random tokens, random-init N(0,0.02) weights",
        "config": {"model": "1B MoE decoder: 16L d2048 16Q/8KV hd128, 8 experts x 2816 top-2, cf 1.25, vocab 32000",
                   "global_batch": c["batch_per_gpu"] * world, "seq_len": c["seq_len"], "parallelism": f"ep{world}",
                   "step": "forward+backward+clip+AdamW (fp32 masters)" + ("" if args.no_graph else ", replayed as one CUDA graph"),
                   "l2": "per-step working set (>5 GB of weights, gradients and activations) exceeds the 126 MB L2",
                   "capacity": "int(1.25*T/E) per expert, whole-token drop in index order (reference rule)",
                   "dp_sync": ("none (one rank)" if world == 1 else
                               "in-switch reduction and multicast stores (multimem over NVLS)"
                               if arena is not None and any(r.mc_grads for r in arena.regions.values())
                               else "reduce-scatter / all-gather by peer loads and stores")},
        "clocks": clocks,
        "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": host[0].numel() * host[0].element_size(), "d2h_bytes_per_step": 4},
        "gpu_launches": launches, "final_loss": loss_dev, "impl": "ours",
    }
    if rank == 0:
        print(json.dumps(res), flush=True)
    if args.kernel_table:
        kernel_table(eager_step, devb, args.kernel_table, rank, world)


def kernel_table(step_fn, batches, path, rank, world):
    """Per-kernel device time of two eagerly launched steps (torch.profiler / CUPTI, outside the timed region):
    rank 0 writes ``name, launches, total_us, avg_us`` sorted by total time, plus the sum, to ``path``. Time a
    kernel spends spinning on a peer's flag is inside its duration, so comparing the table at N=1 and N>1 shows
    where communication is exposed."""
    from torch.profiler import ProfilerActivity, profile

    for i in range(2):
        step_fn(batches[i % len(batches)])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        for i in range(2):
            step_fn(batches[i % len(batches)])
        torch.cuda.synchronize()
    rows = [(e.key, e.count, e.device_time_total) for e in prof.key_averages() if e.device_time_total > 0]
    rows.sort(key=lambda r: -r[2])
    if rank == 0:
        total = sum(r[2] for r in rows)
        with open(path, "w") as f:
            f.write(f"# world={world} steps=2 sum_device_time_us={total:.0f} per_step_us={total / 2:.0f}\n")
            f.write("name\tlaunches\ttotal_us\tavg_us\n")
            for name, n, t in rows:
                f.write(f"{name[:110]}\t{n}\t{t:.0f}\t{t / n:.1f}\n")


def run_reference(args, rank, local, world):
    if world > 1:
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable":
                              "the reference's expert parallelism fails for ep_size>1 (shape error in "
                              "MoEBase.forward after combine, model/moe.py:454-498,1378-1393), so the EP=N config "
                              "cannot run at N>1"}), flush=True)
        return
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "nanopsyche")):
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref/nanopsyche is not installed"}))
        return
    sys.path.insert(0, ref)
    try:
        from nanopsyche.model.moe import MoEBase
        from nanopsyche.model.transformer import Transformer
        from nanopsyche.train.trainer import Trainer, TrainingConfig
    except Exception as e:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"import failed: {type(e).__name__}: {e}"[:300]}))
        return
    dev = torch.device("cuda", local)
    c = CFG
    torch.manual_seed(1234)
    model = Transformer(d_model=c["d_model"], vocab_size=c["vocab"], n_layers=c["n_layers"],
                        block=dict(n_heads=c["n_heads"], n_kv_heads=c["n_kv_heads"], rope_base=c["rope_base"],
                                   max_seq_len=c["seq_len"], qk_norm=False, ffn_hidden=c["ffn_hidden"]))
    for i in range(c["n_layers"]):
        model.replace_block_with_moe_hybrid(i, MoEBase(d_model=c["d_model"], hidden_size=c["moe_hidden"],
                                                       num_experts=c["num_experts"], top_k=c["top_k"],
                                                       capacity_factor=c["capacity_factor"]))
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    model = model.to(dev)
    opt = torch.optim.AdamW(model.parameters(), lr=3e-4, weight_decay=0.1, betas=(0.9, 0.95))
    T = c["batch_per_gpu"] * c["seq_len"]
    tc = TrainingConfig(global_batch_size=T, micro_batch_size=c["batch_per_gpu"], sequence_length=c["seq_len"],
                        max_steps=10 ** 9, dtype=torch.bfloat16, save_interval=10 ** 9, log_interval=10 ** 9)
    n_batches = 4
    torch.manual_seed(99)
    host = [torch.randint(0, c["vocab"], (c["batch_per_gpu"], c["seq_len"])).pin_memory() for _ in range(n_batches)]

    class Loader:  # the reference Trainer calls next() on its loader
        def __init__(self, batches):
            self.batches, self.i = batches, 0

        def __iter__(self):
            return self

        def __next__(self):
            b = self.batches[self.i % len(self.batches)]
            self.i += 1
            return {"input_ids": b, "labels": b}

    devb = [h.to(dev) for h in host]
    trainer = Trainer(tc, model, opt, None, Loader(devb), [])
    trainer.device = dev

    def step(_i):
        trainer._train_step_with_callbacks()

    for i in range(args.warmup):
        step(i)
    sampler = ClockSampler(local)
    sampler.start()
    ms = timed(step, args.steps, 1, dev)
    clocks = sampler.stop()
    trainer.data_loader = Loader(host)  # end to end: batches start in pinned host memory

    def e2e(i):
        trainer._train_step_with_callbacks()
        torch.cuda.synchronize()

    ms_e2e = timed(e2e, args.steps, 1, dev)
    res = {"metric": METRIC, "value": T / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": "bf16 autocast over fp32 weights (the reference's Trainer path)", "data": "synthetic",
           "config": {"model": "1B MoE decoder (same shapes), built with the reference's Transformer + MoEBase",
                      "global_batch": c["batch_per_gpu"], "seq_len": c["seq_len"], "parallelism": "ep1"},
           "clocks": clocks, "e2e": {"value": T / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                                     "h2d_bytes_per_step": host[0].numel() * 8, "d2h_bytes_per_step": 4},
           "impl": "reference"}
    print(json.dumps(res), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a graph")
    ap.add_argument("--kernel-table", default="", help="after the timed runs, write a per-kernel device-time table here")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return 0
    rank, local, world = setup_dist(args.gpus)
    try:
        if args.impl == "reference":
            run_reference(args, rank, local, world)
        else:
            run_ours(args, rank, local, world)
    finally:
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
