"""Command line: ``python -m nanopysche_b200 {train,bench} ...`` (reference: cli.py:20-721).

Same sub-commands and flags as the reference. ``train`` builds the model, parallelises it (the
process group is created when torchrun's ``RANK`` is present), builds the optimizer *after*
parallelisation, and runs the callback-driven ``Trainer``. ``bench`` times full training steps
(forward + backward + optimizer, bf16 on CUDA) with CUDA events on every rank and reports the max
over ranks; ``--forward-only`` reproduces the reference's forward-only timing. Extra flags place MoE
layers (``--moe-interval/--moe-offset/--moe-hidden/--capacity-factor``) and select GQA
(``--n-kv-heads``), which the reference's presets cannot express.
"""
from __future__ import annotations

import argparse
import math
import os
import sys
import time
from typing import Optional

import torch

MODEL_PRESETS = {
    "125m": dict(d_model=768, n_layers=12, n_heads=12, n_kv_heads=12, ffn_hidden=2048),
    "350m": dict(d_model=1024, n_layers=24, n_heads=16, n_kv_heads=16, ffn_hidden=2816),
    "1b": dict(d_model=2048, n_layers=24, n_heads=32, n_kv_heads=32, ffn_hidden=5632),
    "7b": dict(d_model=4096, n_layers=32, n_heads=32, n_kv_heads=32, ffn_hidden=11008),
    # the benchmark shapes: 16 layers, 16 query / 8 KV heads of dim 128
    "1b-gqa": dict(d_model=2048, n_layers=16, n_heads=16, n_kv_heads=8, ffn_hidden=5632, rope_base=10000.0,
                   qk_norm=False),
    "7b-gqa": dict(d_model=4096, n_layers=32, n_heads=32, n_kv_heads=8, ffn_hidden=11008, rope_base=10000.0,
                   qk_norm=False),
}


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="nanopsyche", description="B200-native 5-D parallel training")
    sub = parser.add_subparsers(dest="command", required=True)
    common = argparse.ArgumentParser(add_help=False)
    common.add_argument("--model", choices=sorted(MODEL_PRESETS), default="125m")
    common.add_argument("--use-moe", action="store_true", help="Enable MoE layers")
    common.add_argument("--num-experts", type=int, default=8)
    common.add_argument("--top-k", type=int, default=2)
    common.add_argument("--fp8-recipe", choices=["none", "blockwise", "mxfp8", "flow_moe"], default="none")
    common.add_argument("--fp8-gemm-threshold", type=int, default=1000000)
    common.add_argument("--batch-size", type=int, default=4, help="Micro batch size per GPU")
    common.add_argument("--seq-len", type=int, default=2048)
    common.add_argument("--dataset", type=str, default=None)
    common.add_argument("--device", type=str, default="cuda" if torch.cuda.is_available() else "cpu")
    common.add_argument("--lr", type=float, default=3e-4)
    common.add_argument("--max-steps", type=int, default=100)
    common.add_argument("--model-factory", type=str, default=None)
    common.add_argument("--dtype", choices=["auto", "float32", "bfloat16"], default="auto")
    common.add_argument("--n-kv-heads", type=int, default=None)
    common.add_argument("--moe-interval", type=int, default=2)
    common.add_argument("--moe-offset", type=int, default=0)
    common.add_argument("--moe-hidden", type=int, default=None)
    common.add_argument("--capacity-factor", type=float, default=None)
    common.add_argument("--moe-keep-dense-ffn", action="store_true")
    common.add_argument("--xent-chunk-rows", type=int, default=0,
                        help="head projection and loss over this many rows at a time: the full logits (and their "
                             "gradient) are never formed, at the price of one more head GEMM in the backward pass")
    common.add_argument("--tp-size", type=int, default=1)
    common.add_argument("--async-tp", action="store_true",
                        help="tensor parallelism with the all-gather / reduce-scatter fused into the GEMM kernels "
                             "(sequence-parallel layout over NVLink peer memory)")
    common.add_argument("--sequence-parallel", action="store_true",
                        help="Megatron sequence parallelism under --tp-size: activations between blocks are row shards, "
                             "all-gather / reduce-scatter collectives around the GEMMs (--async-tp fuses them instead)")
    common.add_argument("--pp-size", type=int, default=1)
    common.add_argument("--pp-schedule", default="1F1B", help="GPipe | 1F1B | ZBVZeroBubble | Interleaved1F1B | ...")
    common.add_argument("--pp-microbatches", type=int, default=0, help="microbatches per step (0: one per PP rank)")
    common.add_argument("--cp-size", type=int, default=1)
    common.add_argument("--ep-size", type=int, default=1)
    common.add_argument("--fsdp", action="store_true")
    common.add_argument("--dp-replicate", type=int, default=1,
                        help="hybrid sharding (HSDP): number of replicas of the sharded state; the data-parallel "
                             "ranks split into dp_replicate x dp_shard")
    common.add_argument("--fsdp-backend", choices=["auto", "torch", "arena", "sharded"], default="auto",
                        help="sharded: linear weights sharded by rows, gathered inside their GEMMs (CUDA)")
    common.add_argument("--ac-mode", choices=["full", "selected_blocks"], default=None)
    common.add_argument("--ulysses", action="store_true", help="Ulysses instead of ring attention under CP")
    t = sub.add_parser("train", parents=[common], help="Train a model")
    t.add_argument("--compile", action="store_true")
    t.add_argument("--val-interval", type=int, default=10)      # defaults of the reference's CLI (cli.py:96-135)
    t.add_argument("--val-steps", type=int, default=5)
    t.add_argument("--wandb", action="store_true")
    t.add_argument("--wandb-project", type=str, default="nanopsyche")
    t.add_argument("--resume", type=str, default=None)
    t.add_argument("--save-dir", type=str, default=None, help="default: checkpoints/<model>")
    t.add_argument("--save-interval", type=int, default=1000)
    t.add_argument("--global-batch-size", type=int, default=None, help="tokens per optimizer step")
    t.add_argument("--log-interval", type=int, default=10)
    b = sub.add_parser("bench", parents=[common], help="Benchmark throughput")
    b.add_argument("--warmup", type=int, default=3)
    b.add_argument("--iters", type=int, default=10)
    b.add_argument("--validate", action="store_true")
    b.add_argument("--forward-only", action="store_true")
    return parser


def load_dataset(dataset_spec: Optional[str], batch_size: int, seq_len: int, split: str = "train",
                 val_split: str = "validation", device: str = "cpu"):
    """``(train_loader, val_loader, vocab_size)``; ``None`` loaders mean synthetic tokens."""
    from .train.data import create_distributed_loader

    if dataset_spec is None:
        return None, None, 32000
    if dataset_spec.endswith(".npy") or dataset_spec.endswith(".bin"):
        import numpy as np

        data = np.load(dataset_spec, mmap_mode="r") if dataset_spec.endswith(".npy") else \
            np.memmap(dataset_spec, dtype=np.uint16, mode="r")
        cut = int(len(data) * 0.9)
        return (create_distributed_loader(data[:cut], batch_size, seq_len),
                create_distributed_loader(data[cut:], batch_size, seq_len), 32000)
    try:
        from datasets import load_dataset as hf_load
    except ImportError:
        print("  [data] 'datasets' is not installed: using synthetic tokens")
        return None, None, 32000
    import numpy as np

    ds = hf_load(dataset_spec, split=split, streaming=True)
    try:
        from tokenizers import Tokenizer

        tok = Tokenizer.from_pretrained("gpt2")
        vocab, enc = tok.get_vocab_size(), (lambda s: tok.encode(s).ids)
    except Exception:  # noqa: BLE001
        from transformers import AutoTokenizer

        tk = AutoTokenizer.from_pretrained("gpt2")
        vocab, enc = tk.vocab_size, tk.encode
    tokens: list = []
    for ex in ds:
        text = ex.get("text") or ex.get("content") or ""
        tokens.extend(enc(text[0] if isinstance(text, list) and text else text))
        if len(tokens) >= 1_000_000:
            break
    arr = np.array(tokens[: (len(tokens) // seq_len) * seq_len], dtype=np.int64)
    cut = int(len(arr) * 0.95)
    return (create_distributed_loader(arr[:cut], batch_size, seq_len),
            create_distributed_loader(arr[cut:], batch_size, seq_len), vocab)


@torch.no_grad()
def compute_val_perplexity(model, val_loader, max_batches=10, device=None) -> float:
    """exp(mean loss) over up to ``max_batches`` validation batches, without gradients; arguments in the reference's
    order (cli.py:287), a device given in third place is recognised. A context-parallel model gets
    its share of every sequence (its loss is already the mean over the whole sequence); a pipelined model runs a
    forward-only pass of its schedule and every rank gets the last stage's loss."""
    if not isinstance(max_batches, int):            # (model, val_loader, device[, max_batches])
        max_batches, device = (device if isinstance(device, int) else 10), max_batches
    if device is None:
        device = next(model.parameters()).device
    pp = getattr(model, "_pp_enabled", False)
    stages = (list(model.stages) if hasattr(model, "stages") else [model]) if pp else None
    cp_group = getattr(stages[0] if pp else model, "_cp_group", None)
    model.eval()
    tot, n = 0.0, 0
    it = iter(val_loader)
    sched = None
    with torch.no_grad():
        for _ in range(max_batches):
            try:
                ids, labels = next(it)
            except StopIteration:
                break
            ids, labels, kw = ids.to(device), labels.to(device), {}
            if cp_group is not None:
                import torch.distributed as dist

                from .parallel.context_parallel import shard_batch_for_cp

                ids, labels = shard_batch_for_cp(ids, labels, dist.get_world_size(cp_group), dist.get_rank(cp_group))
                kw["labels_shifted"] = True
            if pp:
                # forward-only pass of the whole pipeline; the loss reaches every rank from the last stage
                from .parallel.pipeline_runtime import PipelineSchedule

                if sched is None or sched.hidden_shape[1] != ids.shape[1]:
                    m = model._pp_config.num_microbatches or model._pp_config.degree
                    m = m if ids.shape[0] % m == 0 else 1
                    sched = PipelineSchedule(stages, model._pp_group, model._pp_config, num_microbatches=m,
                                             hidden_shape=(ids.shape[0] // m, ids.shape[1], stages[0].d_model),
                                             hidden_dtype=next(model.parameters()).dtype)
                tot += float(sched.loss_on_all_ranks(sched.evaluate(ids, target=labels, **kw)))
            else:
                tot += float(model(ids, labels=labels, **kw)["loss"])
            n += 1
    model.train()
    return math.exp(min(tot / max(n, 1), 20.0))


def _resolve_dtype(args) -> torch.dtype:
    if args.dtype == "auto":
        return torch.bfloat16 if str(args.device).startswith("cuda") else torch.float32
    return getattr(torch, args.dtype)


def _model_build_context(args, vocab_size: int):
    from .model_factory import ModelBuildContext

    preset = dict(MODEL_PRESETS[args.model])
    if args.n_kv_heads:
        preset["n_kv_heads"] = args.n_kv_heads
    return ModelBuildContext(vocab_size=vocab_size, seq_len=args.seq_len, device=args.device, model_preset=args.model,
                             preset=preset, use_moe=args.use_moe, num_experts=args.num_experts,
                             moe_top_k=args.top_k, fp8_recipe=args.fp8_recipe,
                             fp8_gemm_threshold=args.fp8_gemm_threshold, dtype=_resolve_dtype(args),
                             moe_interval=args.moe_interval, moe_offset=args.moe_offset, moe_hidden=args.moe_hidden,
                             moe_capacity_factor=args.capacity_factor, moe_keep_dense_ffn=args.moe_keep_dense_ffn)


def _init_distributed(args):
    import torch.distributed as dist

    if "RANK" in os.environ and not dist.is_initialized():
        backend = "nccl" if str(args.device).startswith("cuda") and torch.cuda.is_available() else "gloo"
        if backend == "nccl":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
        dist.init_process_group(backend=backend)
    return dist.get_rank() if dist.is_initialized() else 0, dist.get_world_size() if dist.is_initialized() else 1


def _maybe_parallelize_model(model, args, device):
    """Build the mesh and apply the requested parallelism; returns ``(model, world_mesh | None)``."""
    wants = args.tp_size > 1 or args.pp_size > 1 or args.cp_size > 1 or args.ep_size > 1 or args.fsdp or \
        args.ac_mode is not None
    if not wants:
        return model, None
    from .parallel.context_parallel import ContextParallelConfig
    from .parallel.fsdp import DataParallelConfig
    from .parallel.mesh import build_world_mesh
    from .parallel.pipeline_parallel import PipelineParallelConfig
    from .parallel.tensor_parallel import TensorParallelConfig
    from .parallelize import parallelize_model

    rank, world = _init_distributed(args)
    mesh = None
    if world > 1 or args.fsdp:
        import torch.distributed as dist

        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", "29533")
            dist.init_process_group("gloo" if device.type == "cpu" else "nccl", rank=0, world_size=1)
        rep = max(getattr(args, "dp_replicate", 1), 1)
        hsdp = {}
        if rep > 1:
            dp_total = world // (args.tp_size * args.pp_size * args.cp_size * args.ep_size)
            assert dp_total % rep == 0, "--dp-replicate must divide the data-parallel size"
            hsdp = dict(dp_replicate=rep, dp_shard=dp_total // rep)
        mesh = build_world_mesh(tp_size=args.tp_size, pp_size=args.pp_size, cp_size=args.cp_size,
                                ep_size=args.ep_size, device_type=device.type, replace=True, **hsdp)
    model = parallelize_model(
        model, world_mesh=mesh, device=device,
        tp_config=TensorParallelConfig(args.tp_size, enable_async=getattr(args, "async_tp", False),
                                       sequence_parallel=getattr(args, "async_tp", False) or
                                       getattr(args, "sequence_parallel", False))
        if args.tp_size > 1 else None,
        cp_config=ContextParallelConfig(args.cp_size, ring=not args.ulysses, ulysses=args.ulysses)
        if args.cp_size > 1 else None,
        pp_config=PipelineParallelConfig(args.pp_size, schedule=getattr(args, "pp_schedule", "1F1B"),
                                         num_microbatches=getattr(args, "pp_microbatches", 0) or None)
        if args.pp_size > 1 else None,
        dp_config=DataParallelConfig(param_dtype=_resolve_dtype(args),
                                     backend=getattr(args, "fsdp_backend", "auto")) if args.fsdp else None,
        moe_fp8_recipe=args.fp8_recipe, moe_fp8_gemm_threshold=args.fp8_gemm_threshold,
        compile_model=getattr(args, "compile", False), ac_mode=args.ac_mode) if mesh is not None or args.ac_mode \
        else model
    return model, mesh


def _build_optimizer_and_scheduler(model, args, tokens_per_rank: int, max_steps: int):
    from .engine import prepare_training
    from .train.scheduler import CosineWithWarmup

    pp = getattr(model, "_pp_enabled", False)
    if pp:
        # tokens per forward call of a stage: one pipeline microbatch
        m = getattr(args, "pp_microbatches", 0) or args.pp_size
        tokens_per_rank = tokens_per_rank // max(m, 1)
    if any(getattr(mod, "_tp_fused", False) for mod in model.modules()):
        # fused tensor parallelism keeps activations as row shards between blocks: a MoE layer sees 1 / tp of the rows
        tokens_per_rank = tokens_per_rank // max(getattr(args, "tp_size", 1), 1)
    opt, arena = prepare_training(model, tokens_per_rank=tokens_per_rank, lr=args.lr, weight_decay=0.1,
                                  betas=(0.9, 0.95))
    if pp and arena is not None:
        # the fused optimizer clips by the norm over all pipeline stages: one extra scalar all-reduce on the PP group
        opt.norm_groups = [model._pp_group]
        opt.norm_copies = 2.0 if getattr(model, "is_dualpipe", False) else 1.0
    sched = CosineWithWarmup(opt, warmup_steps=min(10, max(max_steps // 10, 1)), max_steps=max_steps)
    return opt, sched


def cmd_train(args) -> int:
    from .checkpoint.distributed import CheckpointConfig, DistributedCheckpointer
    from .model_factory import build_model
    from .train.callbacks import (ConsoleLoggerCallback, GPUMemoryMonitorCallback, SpeedMonitorCallback,
                                  StabilityMonitorCallback, ValidationCallback, WandBCallback)
    from .train.trainer import Trainer, TrainingConfig

    torch.manual_seed(42)
    args.save_dir = args.save_dir or f"checkpoints/{args.model}"       # the reference's default (cli.py:502)
    rank, world = _init_distributed(args)
    device = torch.device(args.device if not str(args.device).startswith("cuda") else
                          f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}")
    train_loader, val_loader, vocab = load_dataset(args.dataset, args.batch_size, args.seq_len, device=args.device)
    ctx = _model_build_context(args, vocab)
    model, f_opt, f_sched = build_model(ctx, factory_spec=args.model_factory)
    if getattr(args, "xent_chunk_rows", 0) and hasattr(model, "loss_chunk_rows"):
        model.loss_chunk_rows = args.xent_chunk_rows
    model = model.to(device)
    model, mesh = _maybe_parallelize_model(model, args, device)
    if getattr(args, "compile", False) and mesh is None and hasattr(model, "apply_compile"):
        model.apply_compile()
    dp = max(world // (args.tp_size * args.pp_size * args.cp_size), 1)
    if f_opt is None:
        opt, sched = _build_optimizer_and_scheduler(model, args, args.batch_size * args.seq_len // args.cp_size,
                                                    args.max_steps)
    else:
        opt, sched = f_opt, f_sched
    gbs = args.global_batch_size or args.batch_size * args.seq_len * dp
    tc = TrainingConfig(global_batch_size=gbs, micro_batch_size=args.batch_size, sequence_length=args.seq_len,
                        learning_rate=args.lr, max_steps=args.max_steps, dtype=torch.bfloat16, save_dir=args.save_dir,
                        save_interval=args.save_interval, log_interval=args.log_interval, dp_world_size=dp,
                        vocab_size=vocab, cp_size=args.cp_size, pp_schedule=args.pp_schedule,
                        pp_microbatches=args.pp_microbatches)
    ckpt = DistributedCheckpointer(CheckpointConfig(save_dir=args.save_dir, save_interval=args.save_interval or 10**9))
    callbacks = [SpeedMonitorCallback(device=device), StabilityMonitorCallback(), ConsoleLoggerCallback(log_interval=1)]
    if device.type == "cuda":
        callbacks.insert(1, GPUMemoryMonitorCallback(device))
    from .train.callbacks import ThroughputSummaryCallback

    callbacks.append(ThroughputSummaryCallback(
        warmup_steps=min(5, max(args.max_steps // 3, 1)),
        label={"model": args.model, "tp": args.tp_size, "pp": args.pp_size, "cp": args.cp_size, "ep": args.ep_size,
               "batch": args.batch_size, "seq": args.seq_len}))
    if args.wandb:
        callbacks.append(WandBCallback(project=args.wandb_project, config=vars(args)))
    if args.val_interval and val_loader is not None:
        callbacks.append(ValidationCallback(lambda: compute_val_perplexity(model, val_loader, device, args.val_steps),
                                            args.val_interval))
    trainer = Trainer(tc, model, opt, sched, train_loader, callbacks, ckpt, device=device)
    if args.resume:
        step = trainer.load_checkpoint(args.resume)
        if rank == 0:
            print(f"resumed from {args.resume} at step {step}")
    if rank == 0:
        n = sum(p.numel() for p in model.parameters())
        print(f"model={args.model} params={n / 1e6:.1f}M device={device} world={world} accum="
              f"{tc.gradient_accumulation_steps}")
    trainer.fit()
    if args.save_interval:
        ckpt.save(trainer.step, model, opt, scheduler=sched)
    return 0


def cmd_bench(args) -> int:
    from .bench_utils import compute_mfu
    from .model_factory import build_model

    torch.manual_seed(42)
    rank, world = _init_distributed(args)
    device = torch.device(args.device if not str(args.device).startswith("cuda") else
                          f"cuda:{int(os.environ.get('LOCAL_RANK', 0))}")
    _, val_loader, vocab = load_dataset(args.dataset, args.batch_size, args.seq_len, device=args.device)
    ctx = _model_build_context(args, vocab)
    model, _, _ = build_model(ctx, factory_spec=args.model_factory)
    if getattr(args, "xent_chunk_rows", 0) and hasattr(model, "loss_chunk_rows"):
        model.loss_chunk_rows = args.xent_chunk_rows
    model = model.to(device)
    model, _ = _maybe_parallelize_model(model, args, device)
    model.train()
    opt = None
    if not args.forward_only:
        opt, _ = _build_optimizer_and_scheduler(model, args, args.batch_size * args.seq_len // args.cp_size, 1000)
    x = torch.randint(0, vocab, (args.batch_size, args.seq_len), device=device)
    labels, fwd_kw = x, {}
    cp_group = getattr(model, "_cp_group", None) or getattr(getattr(model, "stages", [None])[0], "_cp_group", None)
    if cp_group is not None:           # every context-parallel rank works on its share of each sequence
        import torch.distributed as dist

        from .parallel.context_parallel import shard_batch_for_cp

        x, labels = shard_batch_for_cp(x, x, dist.get_world_size(cp_group), dist.get_rank(cp_group))
        fwd_kw["labels_shifted"] = True
    sched = None
    if getattr(model, "_pp_enabled", False):
        # a pipeline stage is stepped by the schedule executor (forward and backward of all micro-batches)
        import torch.distributed as dist

        from .parallel.pipeline_runtime import PipelineSchedule

        if args.forward_only:
            raise SystemExit("bench --forward-only is not available with --pp-size > 1: a pipeline step is a full step")
        stages = list(model.stages) if hasattr(model, "stages") else [model]
        m = getattr(args, "pp_microbatches", 0) or args.pp_size
        assert args.batch_size % m == 0, "--batch-size must be a multiple of the pipeline micro-batch count"
        sched = PipelineSchedule(stages, model._pp_group, model._pp_config, num_microbatches=m,
                                 hidden_shape=(args.batch_size // m, x.shape[1], stages[0].d_model),
                                 hidden_dtype=next(model.parameters()).dtype)

    def step():
        if sched is not None:
            sched.step(x, target=labels, **fwd_kw)
            if getattr(model, "is_dualpipe", False):      # the two copies of every stage exchange their gradient halves
                from .parallel.pipeline_runtime import sync_twin_grads

                arena_opt = type(opt).__name__ == "ArenaAdamW"
                sync_twin_grads(list(model.stages), model._pp_group,
                                grad_of=(lambda q: getattr(q, "main_grad", None)) if arena_opt else None)
            opt.step()
            opt.zero_grad(set_to_none=True)
            return
        if args.forward_only:
            with torch.no_grad():
                model(x)
            return
        out = model(x, labels=labels, **fwd_kw)
        loss = out["loss"] if out.get("aux_loss") is None else out["loss"] + out["aux_loss"]
        loss.backward()
        opt.step()
        opt.zero_grad(set_to_none=True)

    for _ in range(args.warmup):
        step()
    if device.type == "cuda":
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(args.iters):
            step()
        e.record()
        torch.cuda.synchronize()
        elapsed = s.elapsed_time(e) / 1e3
    else:
        t0 = time.time()
        for _ in range(args.iters):
            step()
        elapsed = time.time() - t0
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([elapsed], device=device if device.type == "cuda" else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed = float(t)
    dp = max(world // (args.tp_size * args.pp_size * args.cp_size), 1)
    tokens = args.batch_size * args.seq_len * args.iters * dp
    tps = tokens / elapsed
    p = MODEL_PRESETS[args.model]
    mfu = compute_mfu(elapsed / args.iters, p["n_layers"], p["d_model"], args.moe_hidden or p["ffn_hidden"],
                      p["n_heads"], args.seq_len, args.batch_size * dp, device=device, num_gpus=world,
                      num_experts=args.num_experts if args.use_moe else 0, top_k=args.top_k if args.use_moe else 0)
    if args.forward_only:
        mfu /= 3.0
    if rank == 0:
        n = sum(q.numel() for q in model.parameters())
        print(f"params: {n / 1e6:.1f}M | mode: {'forward' if args.forward_only else 'train step'}")
        print(f"time/step: {1e3 * elapsed / args.iters:.2f} ms | tokens/s: {tps:,.0f} | per GPU: {tps / world:,.0f} "
              f"| MFU: {100 * mfu:.1f}%")
        if args.validate and val_loader is not None:
            print(f"val perplexity: {compute_val_perplexity(model, val_loader, device):.2f}")
    return 0


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    return cmd_train(args) if args.command == "train" else cmd_bench(args)


if __name__ == "__main__":
    sys.exit(main())
