"""Headline benchmark: training tokens/s of the 1B MoE decoder with expert parallelism over all GPUs.

    python bench.py --gpus N --steps K --warmup W            (N > 1: launched once per rank by torchrun)
    python bench.py --impl reference ...                     the unmodified reference from baseline/_ref
    python bench.py --impl baseline ...                      this repository's model on library calls only

Config (per GPU batch 2 x seq 2048, weak scaling): 16 layers, d_model 2048, 16 query / 8 KV heads of
dim 128, every FFN replaced by 8 SwiGLU experts (hidden 2816), top-2 softmax routing with the
DeepSeek-V3 auxiliary-loss-free bias, capacity factor 1.25, vocab 32000, RoPE base 10000, random-init
N(0, 0.02) weights, uniform random tokens, bf16 compute with fp32 master weights, EP = N; FP8-Flow-MoE
recipe (e4m3, 1x128 activation / 128x128 weight scales) for the expert GEMMs once a local expert sees at
least ``--fp8-gemm-threshold`` tokens. One step = forward + backward + gradient clipping + AdamW +
learning-rate schedule (the reference CLI's: linear warm-up over min(10, max_steps // 10) steps, then
cosine; cli.py:362-366).

Arms:
  ours       the fused sm_100a path (one CUDA graph per step), EP = N over peer memory
  reference  the unmodified reference package: its Transformer + MoEBase + Trainer. At N > 1 its expert
             parallelism raises a shape error, so the arm drives the multi-GPU path it does have for this
             model, ``Transformer.apply_fsdp`` (FSDP2 full shard, every rank holds all experts' shards)
  baseline   this repository's model with every op on its PyTorch statement (cuBLAS, SDPA, ATen), experts as
             per-expert matmuls behind the NCCL all-to-all dispatcher, ``torch.optim.AdamW`` and an NCCL
             all-reduce of the replicated gradients: the un-fused arm the fused kernels are measured against

Learning rate: 3e-5 in every arm. The architecture is the reference's (no norm in front of the LM head, every
matrix N(0, 0.02)): the residual stream leaves 16 blocks with entries of order 1, so the first loss is 13.3 rather
than ln(32000) = 10.4 in all three arms, and at the reference CLI's default of 3e-4 the loss of all three arms
climbs to 30 and beyond within 20 steps (measured: fused 36.3, reference 29.8, plain baseline 36.1). At 3e-5 it
falls steadily (13.3 -> 9.4 in 70 steps with four cycled batches), which is what a timed step should be doing.

Timing: W untimed steps, then exactly K steps between CUDA events with a barrier + synchronize on both
sides, max over ranks; the end-to-end figure repeats the K steps with a pinned-host -> device copy of the
tokens and a device -> host read of the loss inside every step. GPU clocks and throttle reasons are
sampled with nvidia-smi during the timed region.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
CFG = dict(n_layers=16, d_model=2048, n_heads=16, n_kv_heads=8, ffn_hidden=5632, moe_hidden=2816, num_experts=8,
           top_k=2, capacity_factor=1.25, vocab=32000, batch_per_gpu=2, seq_len=2048, rope_base=10000.0)
TINY = dict(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, ffn_hidden=128, moe_hidden=64, num_experts=4,
            top_k=2, capacity_factor=1.25, vocab=512, batch_per_gpu=2, seq_len=32, rope_base=10000.0)
METRIC = "tokens/s (device-timed, max over ranks) 1B MoE EP8 at 1/2/4/8 B200 vs ref NCCL"
LR, WD, BETAS, CLIP = 3e-5, 0.1, (0.9, 0.95), 1.0   # lr: see the note on stability in the module docstring
NOMINAL_MAX_STEPS = 10000                       # run length the schedule is laid out for
LR_WARMUP = min(10, NOMINAL_MAX_STEPS // 10)    # the reference CLI's rule
N_BATCHES = 2                                   # fixed random batches, cycled
WARM = [LR_WARMUP]                              # warm-up steps in use (``--lr-warmup`` overrides)

# Tokens/s of the plain library-call arm (``--impl baseline``) measured on this pool's B200s with the command in
# the module docstring; ``vs_baseline`` of the fused arm divides by the entry for its N. None: not measured.
BASELINE_ARM_TOKENS_PER_S = {1: 19156.0, 2: 27482.0, 4: 70985.0, 8: 167488.0}


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


def setup_dist():
    rank = int(os.environ.get("RANK", 0))
    local = int(os.environ.get("LOCAL_RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    cuda = torch.cuda.is_available()
    if cuda:
        torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if cuda:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        else:
            os.environ.setdefault("GLOO_SOCKET_IFNAME", "lo")
            dist.init_process_group("gloo")
    return rank, local, world, torch.device("cuda", local) if cuda else torch.device("cpu")


def timed(step_fn, steps: int, world: int, dev):
    """ms per step: device-timed with CUDA events (wall clock on a CPU dry run), max over ranks."""
    cuda = dev.type == "cuda"
    if world > 1:
        dist.barrier()
    if cuda:
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
    else:
        import time

        t0 = time.perf_counter()
    for i in range(steps):
        step_fn(i)
    if cuda:
        e.record()
        torch.cuda.synchronize()
        el = s.elapsed_time(e)
    else:
        el = (time.perf_counter() - t0) * 1e3
    if world > 1:
        dist.barrier()
    ms = torch.tensor([el], device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    return float(ms) / steps


def make_batches(c, rank, dev):
    torch.manual_seed(99 + rank)
    host = [torch.randint(0, c["vocab"], (c["batch_per_gpu"], c["seq_len"])) for _ in range(N_BATCHES)]
    if dev.type == "cuda":
        host = [h.pin_memory() for h in host]
    return host, [h.to(dev) for h in host]


def mean_over_ranks(x: float, world: int, dev) -> float:
    if world <= 1:
        return float(x)
    t = torch.tensor([float(x)], device=dev, dtype=torch.float64 if dev.type == "cpu" else torch.float32)
    dist.all_reduce(t)
    return float(t) / world


def result_line(args, *, c, world, ms, ms_e2e, clocks, impl, dtype, model_desc, parallelism, host, extra_cfg=None,
                **more):
    T = c["batch_per_gpu"] * c["seq_len"]
    tokens = T * world
    cfg = {"model": model_desc, "global_batch": c["batch_per_gpu"] * world, "seq_len": c["seq_len"],
           "parallelism": parallelism,
           "schedule": f"AdamW lr {LR} betas {BETAS} wd {WD}, clip {CLIP}, linear warm-up {WARM[0]} steps then cosine",
           "l2": "per-step working set (>5 GB of weights, gradients and activations) exceeds the 126 MB L2"}
    cfg.update(extra_cfg or {})
    if c is not CFG:
        cfg["model"] = "toy-sized dry run of the harness (--tiny): " + json.dumps(c)
    res = {"metric": METRIC, "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
           "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
           "dtype": dtype, "data": "synthetic uniform random tokens, random-init N(0,0.02) weights", "config": cfg,
           "clocks": clocks,
           "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "ms_per_step": ms_e2e,
                   "h2d_bytes_per_step": host[0].numel() * host[0].element_size(), "d2h_bytes_per_step": 4},
           "impl": impl}
    res.update(more)
    return res


# ---------------------------------------------------------------------------------------------------- fused arm
def run_ours(args, rank, local, world, dev, c):
    sys.path.insert(0, ROOT)
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.engine import GraphedTrainStep, prepare_training
    from nanopysche_b200.models.moe import ExpertParallelConfig
    from nanopysche_b200.ops import _lib
    from nanopysche_b200.train.scheduler import CosineWithWarmup

    cuda = dev.type == "cuda"
    recipe = args.fp8_recipe
    cfg = TransformerConfig(vocab_size=c["vocab"], d_model=c["d_model"], n_layers=c["n_layers"], n_heads=c["n_heads"],
                            n_kv_heads=c["n_kv_heads"], ffn_hidden=c["ffn_hidden"], rope_base=c["rope_base"],
                            max_seq_len=c["seq_len"], qk_norm=False, use_moe=True, num_experts=c["num_experts"],
                            moe_top_k=c["top_k"], moe_interval=1, moe_offset=0, moe_hidden=c["moe_hidden"],
                            moe_capacity_factor=c["capacity_factor"], moe_bias_gamma=args.bias_gamma or None,
                            fp8_flow_moe=recipe != "none", fp8_recipe=recipe,
                            fp8_gemm_threshold=args.fp8_gemm_threshold)
    torch.manual_seed(1234)  # identical replicated weights on every rank
    model = cfg.build(dtype=torch.bfloat16 if cuda else torch.float32, init_device=str(dev) if cuda else "cpu")
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    if world > 1:
        model.apply_ep(ExpertParallelConfig(ep_size=world, ep_group=dist.group.WORLD))
        model._needs_grad_sync = True
    T = c["batch_per_gpu"] * c["seq_len"]
    opt, arena = prepare_training(model, tokens_per_rank=T, lr=LR, weight_decay=WD, max_grad_norm=CLIP,
                                  dp_group=dist.group.WORLD if world > 1 else None,
                                  ep_group=dist.group.WORLD if world > 1 else None)
    sched = CosineWithWarmup(opt, warmup_steps=WARM[0], max_steps=NOMINAL_MAX_STEPS)
    model.train()
    host, devb = make_batches(c, rank, dev)
    last, trace = {}, []

    def eager_step(ids):
        out = model(ids, labels=ids)
        loss = out["loss"] if out.get("aux_loss") is None else out["loss"] + out["aux_loss"]
        loss.backward()
        if arena is None:
            if world > 1:
                for p in model.parameters():
                    if p.grad is not None and not getattr(p, "_ep_sharded", False):
                        dist.all_reduce(p.grad)
                        p.grad.div_(world)
            torch.nn.utils.clip_grad_norm_(model.parameters(), CLIP)
        opt.step()
        opt.zero_grad(set_to_none=True)
        last["loss"] = out["loss"].detach()

    graphed, per_step = None, 0
    if cuda and not args.no_graph:
        # the whole step (forward + backward + clip + AdamW) replayed as one CUDA graph; its two eager warm-up
        # steps run at the schedule's first learning rate (0)
        l0 = _lib.LAUNCHES
        graphed = GraphedTrainStep(model, opt, devb[0], warmup=2).capture()
        per_step = (_lib.LAUNCHES - l0) // 3  # two eager warm-up steps + the captured one

    def train_step(ids):
        if graphed is not None:
            last["loss"] = graphed.step(ids)
        else:
            eager_step(ids)
        sched.step()
        if args.trace_loss:
            trace.append(last["loss"].clone())

    train_step(devb[0])
    first_loss = float(last["loss"])
    for i in range(1, args.warmup):
        train_step(devb[i % N_BATCHES])
    if cuda:
        torch.cuda.synchronize()
        _lib.check_status("after warm-up")
        _lib.wait_stats(reset=True)
    sampler = ClockSampler(local)
    if rank == 0 and cuda:
        sampler.start()
    l0 = _lib.LAUNCHES
    ms = timed(lambda i: train_step(devb[i % N_BATCHES]), args.steps, world, dev)
    launches = (_lib.LAUNCHES - l0) if graphed is None else per_step * args.steps
    clocks = sampler.stop() if (rank == 0 and cuda) else {}
    exposed = None
    if cuda:
        ws = _lib.wait_stats(reset=True)
        exposed = mean_over_ranks(ws["exposed_ms"] / args.steps, world, dev) if ws is not None else None

    def e2e_step(i):
        ids = host[i % N_BATCHES]
        train_step(ids if graphed is not None else ids.to(dev, non_blocking=True))  # graph: copied into its static input
        last["host_loss"] = last["loss"].item()

    ms_e2e = timed(e2e_step, args.steps, world, dev)
    if cuda:
        _lib.check_status("after timed region")
    final_loss = mean_over_ranks(float(last["loss"]), world, dev)
    first_loss = mean_over_ranks(first_loss, world, dev)
    rt = next((m._fused_runtime for m in model.modules() if getattr(m, "_fused_runtime", None) is not None), None)
    fp8_on = bool(rt is not None and rt.fp8)
    res = result_line(
        args, c=c, world=world, ms=ms, ms_e2e=ms_e2e, clocks=clocks, impl="ours", host=host,
        dtype="bf16 + e4m3 experts (fp32 masters)" if fp8_on else "bf16",
        model_desc="1B MoE decoder: 16L d2048 16Q/8KV hd128, 8 experts x 2816 top-2, cf 1.25, vocab 32000",
        parallelism=f"ep{world}",
        extra_cfg={"step": "forward+backward+clip+AdamW (fp32 masters)" +
                           ("" if graphed is None else ", replayed as one CUDA graph"),
                   "capacity": "int(1.25*T/E) per expert, whole-token drop in index order (reference rule)",
                   "router_bias": f"DeepSeek-V3 aux-free bias, gamma {args.bias_gamma}, updated on the device every step"
                   if args.bias_gamma else "off",
                   "fp8_recipe": f"{recipe}, threshold {args.fp8_gemm_threshold} tokens/expert: "
                                 f"{'fp8 expert GEMMs' if fp8_on else 'below threshold, bf16 expert GEMMs'}"
                   if recipe != "none" else "none",
                   "dp_sync": ("none (one rank)" if world == 1 else
                               "in-switch reduction and multicast stores (multimem over NVLS)"
                               if arena is not None and any(r.mc_grads for r in arena.regions.values())
                               else "reduce-scatter / all-gather by peer loads and stores")},
        gpu_launches=launches, first_loss=first_loss, final_loss=final_loss, exposed_comm_ms=exposed)
    base = BASELINE_ARM_TOKENS_PER_S.get(world)
    if base and c is CFG:
        res["vs_baseline"] = res["value"] / base
    if rank == 0:
        print(json.dumps(res), flush=True)
        if args.trace_loss:
            print("loss trace:", [round(float(x), 3) for x in trace], file=sys.stderr, flush=True)
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


# ------------------------------------------------------------------------------------------- plain library arm
def run_baseline(args, rank, local, world, dev, c):
    """This repository's model with every op on its PyTorch statement: fp32 weights under bf16 autocast, cuBLAS
    linears, SDPA attention, per-expert matmuls behind ``NcclAllToAllDispatcher``, ``torch.optim.AdamW``, one flat
    NCCL all-reduce of the replicated gradients and ``clip_grad_norm_``-style clipping over all ranks' shards."""
    sys.path.insert(0, ROOT)
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.models.moe import ExpertParallelConfig, NcclAllToAllDispatcher
    from nanopysche_b200.ops import _lib
    from nanopysche_b200.train.scheduler import CosineWithWarmup

    _lib.set_plain(True)
    cuda = dev.type == "cuda"
    cfg = TransformerConfig(vocab_size=c["vocab"], d_model=c["d_model"], n_layers=c["n_layers"], n_heads=c["n_heads"],
                            n_kv_heads=c["n_kv_heads"], ffn_hidden=c["ffn_hidden"], rope_base=c["rope_base"],
                            max_seq_len=c["seq_len"], qk_norm=False, use_moe=True, num_experts=c["num_experts"],
                            moe_top_k=c["top_k"], moe_interval=1, moe_offset=0, moe_hidden=c["moe_hidden"],
                            moe_capacity_factor=c["capacity_factor"], moe_bias_gamma=args.bias_gamma or None)
    torch.manual_seed(1234)
    model = cfg.build(dtype=torch.float32, init_device=str(dev) if cuda else "cpu")
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.normal_(0.0, 0.02)
    if world > 1:
        model.apply_ep(ExpertParallelConfig(ep_size=world, ep_group=dist.group.WORLD,
                                            dispatcher=NcclAllToAllDispatcher()))
    repl = [p for p in model.parameters() if not getattr(p, "_ep_sharded", False)]
    shard = [p for p in model.parameters() if getattr(p, "_ep_sharded", False)]
    opt = torch.optim.AdamW(model.parameters(), lr=LR, betas=BETAS, weight_decay=WD, fused=cuda)
    sched = CosineWithWarmup(opt, warmup_steps=WARM[0], max_steps=NOMINAL_MAX_STEPS)
    routers = [m for m in model.modules() if hasattr(m, "post_batch") and getattr(m, "score_bias", None) is not None]
    model.train()
    host, devb = make_batches(c, rank, dev)
    last = {}

    def step(ids):
        with torch.autocast(device_type=dev.type, dtype=torch.bfloat16):
            out = model(ids, labels=ids)
            loss = out["loss"] if out.get("aux_loss") is None else out["loss"] + out["aux_loss"]
        loss.backward()
        if world > 1:
            flat = torch._utils._flatten_dense_tensors([p.grad for p in repl])
            dist.all_reduce(flat)
            flat.div_(world)
            for p, g in zip(repl, torch._utils._unflatten_dense_tensors(flat, [p.grad for p in repl])):
                p.grad.copy_(g)
        sq = torch.stack([p.grad.float().pow(2).sum() for p in shard]).sum() if shard else torch.zeros((), device=dev)
        if world > 1:
            dist.all_reduce(sq)
        sq = sq + torch.stack([p.grad.float().pow(2).sum() for p in repl]).sum()
        coef = torch.clamp(CLIP / (sq.sqrt() + 1e-6), max=1.0)
        torch._foreach_mul_([p.grad for p in model.parameters() if p.grad is not None], coef)
        opt.step()
        opt.zero_grad(set_to_none=True)
        for r in routers:
            r.post_batch()
        sched.step()
        last["loss"] = out["loss"].detach()

    step(devb[0])
    first_loss = mean_over_ranks(float(last["loss"]), world, dev)
    for i in range(1, args.warmup):
        step(devb[i % N_BATCHES])
    sampler = ClockSampler(local)
    if rank == 0 and cuda:
        sampler.start()
    ms = timed(lambda i: step(devb[i % N_BATCHES]), args.steps, world, dev)
    clocks = sampler.stop() if (rank == 0 and cuda) else {}

    def e2e(i):
        step(host[i % N_BATCHES].to(dev, non_blocking=True))
        last["host_loss"] = last["loss"].item()

    ms_e2e = timed(e2e, args.steps, world, dev)
    res = result_line(
        args, c=c, world=world, ms=ms, ms_e2e=ms_e2e, clocks=clocks, impl="baseline", host=host,
        dtype="bf16 autocast over fp32 weights",
        model_desc="1B MoE decoder (same shapes and routing), this repository's model on PyTorch library ops",
        parallelism=f"ep{world} (NCCL all-to-all dispatcher, NCCL all-reduce of replicated gradients)",
        first_loss=first_loss, final_loss=mean_over_ranks(float(last["loss"]), world, dev), gpu_launches=0)
    if rank == 0:
        print(json.dumps(res), flush=True)


# ------------------------------------------------------------------------------------------------ reference arm
def build_reference(c, dev, world):
    """The reference's own model for the benchmark shapes, its optimizer, schedule and Trainer. Returns
    ``(trainer, losses)``; ``losses`` collects the loss the Trainer records at every step."""
    from nanopsyche.model.moe import MoEBase
    from nanopsyche.model.transformer import Transformer
    from nanopsyche.train.callbacks.base import Callback
    from nanopsyche.train.scheduler import CosineWithWarmup
    from nanopsyche.train.trainer import Trainer, TrainingConfig

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
    if world > 1:
        # the reference's stock multi-GPU path for this model (model/transformer.py:302-338,570-627)
        from torch.distributed.device_mesh import init_device_mesh

        mesh = init_device_mesh(dev.type, (world,), mesh_dim_names=("dp",))
        model.apply_fsdp(dp_mesh=mesh)
    opt = torch.optim.AdamW(model.parameters(), lr=LR, weight_decay=WD, betas=BETAS)   # after sharding
    sched = CosineWithWarmup(opt, warmup_steps=WARM[0], max_steps=NOMINAL_MAX_STEPS)
    T = c["batch_per_gpu"] * c["seq_len"]
    tc = TrainingConfig(global_batch_size=T, micro_batch_size=c["batch_per_gpu"], sequence_length=c["seq_len"],
                        max_steps=10 ** 9, dtype=torch.bfloat16, save_interval=10 ** 9, log_interval=10 ** 9)
    losses = []

    class LossTap(Callback):  # the Trainer's own metric, read at the hook that follows forward + backward
        def post_train_batch(self, trainer):
            losses.append(trainer._metrics.get("train/CE loss"))

    trainer = Trainer(tc, model, opt, sched, None, [LossTap()])
    trainer.device = dev
    # fit() counts steps itself; the stand-alone step call reads ``trainer.step`` for its rank-0-only metric flush
    # (a collective the other ranks never enter) and its checkpoint trigger: a step number off both intervals
    trainer.step = 1
    return trainer, losses


class CyclingLoader:
    """The reference Trainer calls ``next()`` on its loader."""

    def __init__(self, batches):
        self.batches, self.i = batches, 0

    def __iter__(self):
        return self

    def __next__(self):
        b = self.batches[self.i % len(self.batches)]
        self.i += 1
        return {"input_ids": b, "labels": b}


def run_reference(args, rank, local, world, dev, c):
    def unavailable(why):
        if rank == 0:
            print(json.dumps({"impl": "reference", "unavailable": why[:300]}), flush=True)

    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "nanopsyche")):
        return unavailable("baseline/_ref/nanopsyche is not installed")
    sys.path.insert(0, ref)
    try:
        trainer, losses = build_reference(c, dev, world)
    except Exception as e:  # noqa: BLE001
        return unavailable(f"building the reference model failed: {type(e).__name__}: {e}")
    cuda = dev.type == "cuda"
    host, devb = make_batches(c, rank, dev)
    trainer.data_loader = CyclingLoader(devb)

    def step(_i):
        trainer._train_step_with_callbacks()

    import contextlib
    import io

    quiet = contextlib.redirect_stdout(io.StringIO())   # the Trainer prints a line per step
    with quiet:
        for i in range(args.warmup):
            step(i)
        sampler = ClockSampler(local)
        if rank == 0 and cuda:
            sampler.start()
        ms = timed(step, args.steps, world, dev)
        clocks = sampler.stop() if (rank == 0 and cuda) else {}
        trainer.data_loader = CyclingLoader(host)  # end to end: batches start in pinned host memory

        def e2e(i):
            trainer._train_step_with_callbacks()
            if cuda:
                torch.cuda.synchronize()

        ms_e2e = timed(e2e, args.steps, world, dev)
    vals = [x for x in losses if x is not None]
    res = result_line(
        args, c=c, world=world, ms=ms, ms_e2e=ms_e2e, clocks=clocks, impl="reference", host=host,
        dtype="bf16 autocast over fp32 weights (the reference's Trainer path)",
        model_desc="1B MoE decoder (same shapes), built with the reference's Transformer + MoEBase",
        parallelism="ep1" if world == 1 else
        f"fsdp{world} (the reference's expert parallelism raises for ep_size > 1; Transformer.apply_fsdp is its "
        "multi-GPU path for this model)",
        first_loss=mean_over_ranks(vals[0], world, dev) if vals else None,
        final_loss=mean_over_ranks(vals[-1], world, dev) if vals else None,
        extra_cfg={"loss": "the Trainer's 'train/CE loss' metric (cross-entropy + auxiliary loss)"})
    res["e2e"]["h2d_bytes_per_step"] = host[0].numel() * 8
    if rank == 0:
        print(json.dumps(res), flush=True)


def main():
    global LR
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference", "baseline"], default="ours")
    ap.add_argument("--fp8-recipe", choices=["none", "blockwise", "flow_moe"], default="flow_moe")
    ap.add_argument("--fp8-gemm-threshold", type=int, default=2048, help="tokens per local expert from which the "
                    "expert GEMMs run in fp8")
    ap.add_argument("--bias-gamma", type=float, default=1e-3, help="DeepSeek-V3 router bias update rate (0: off)")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a graph")
    ap.add_argument("--kernel-table", default="", help="after the timed runs, write a per-kernel device-time table here")
    ap.add_argument("--trace-loss", action="store_true", help="print the loss of every step to stderr")
    ap.add_argument("--lr", type=float, default=LR, help="peak learning rate")
    ap.add_argument("--lr-warmup", type=int, default=LR_WARMUP, help="learning-rate warm-up steps (0: constant lr)")
    ap.add_argument("--tiny", action="store_true", help="a toy-sized model (dry run of the harness; also runs on CPU)")
    args = ap.parse_args()
    if not torch.cuda.is_available() and not args.tiny:
        print(json.dumps({"impl": args.impl, "unavailable": "no CUDA device visible"}))
        return 0
    args.warmup = max(args.warmup, 1)
    WARM[0] = args.lr_warmup
    LR = args.lr
    rank, local, world, dev = setup_dist()
    c = TINY if args.tiny else CFG
    try:
        {"ours": run_ours, "reference": run_reference, "baseline": run_baseline}[args.impl](args, rank, local, world,
                                                                                            dev, c)
    finally:
        if world > 1 and dist.is_initialized():
            dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
