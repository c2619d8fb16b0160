"""Runs the unmodified reference (installed under ``baseline/_ref``) on small CPU cases and writes what it computed
to a file: ``python tests/reference_oracle.py out.pt``. ``tests/test_reference_parity_cpu.py`` loads the same weights
and inputs into this package and compares. It is a separate process because the reference's top-level package name
(``nanopsyche``) is the name of this repository's alias package.

Nothing of this package is imported here."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

BASE = dict(d_model=64, vocab_size=128, n_layers=2)
BLOCK = dict(n_heads=4, n_kv_heads=2, rope_base=10000.0, max_seq_len=64, ffn_hidden=128)
MOE = dict(d_model=64, hidden_size=96, num_experts=4, top_k=2)

# name -> (Transformer kwargs, block kwargs, MoEBase kwargs or None); enum values by name
MODEL_CASES = {
    "dense": ({}, dict(qk_norm=False), None),
    "dense_qk_norm": ({}, dict(qk_norm=True), None),
    "dense_tied": (dict(tie_word_embeddings=True), dict(qk_norm=False), None),
    "dense_mha_head_dim": ({}, dict(qk_norm=False, n_kv_heads=4, head_dim=32), None),
    "dense_dropout": ({}, dict(qk_norm=False, dropout=0.1), None),
    "dense_embedding_norm": (dict(embedding_norm="RMSNorm"), dict(qk_norm=True), None),
    "moe": ({}, dict(qk_norm=False), {}),
    "moe_capacity_1": ({}, dict(qk_norm=False), dict(capacity_factor=1.0)),
    "moe_capacity_1p25": ({}, dict(qk_norm=False), dict(capacity_factor=1.25)),
    "moe_sigmoid": ({}, dict(qk_norm=False), dict(gating_function="SIGMOID")),
    "moe_z_loss": ({}, dict(qk_norm=False), dict(z_loss_multiplier=1e-3)),
    "moe_gate_bias": ({}, dict(qk_norm=False), dict(bias=True)),
    "moe_shared_expert": ({}, dict(qk_norm=False), dict(shared_expert=True)),
    "moe_score_bias": ({}, dict(qk_norm=False), dict(bias_gamma=1e-2)),
    "moe_top1_8_experts": ({}, dict(qk_norm=False), dict(num_experts=8, top_k=1, capacity_factor=1.5)),
}


def build(transformer_cls, moe_module, case, seed=0):
    tkw, bkw, mkw = MODEL_CASES[case]
    tkw = dict(tkw)
    if tkw.get("embedding_norm") == "RMSNorm":       # the norm class that the Transformer's own module uses
        tkw["embedding_norm"] = getattr(sys.modules[transformer_cls.__module__], "RMSNorm")(BASE["d_model"])
    torch.manual_seed(seed)
    model = transformer_cls(**BASE, **tkw, block=dict(BLOCK, **bkw))
    if mkw is not None:
        kw = dict(MOE, **mkw)
        if "gating_function" in kw:
            kw["gating_function"] = getattr(moe_module.GatingFunction, kw["gating_function"])
        for i in range(BASE["n_layers"]):
            model.replace_block_with_moe_hybrid(i, moe_module.MoEBase(**kw))
    return model


def run_model(model, ids):
    model.train()
    torch.manual_seed(3)                     # dropout masks of the case that has dropout
    out = model(ids, labels=ids)
    out["loss"].backward()
    return {"keys": sorted(out.keys()), "logits": out["logits"].detach(), "loss": out["loss"].detach(),
            "aux_loss": None if out.get("aux_loss") is None else out["aux_loss"].detach(),
            "grads": {n: p.grad.detach().clone() for n, p in model.named_parameters() if p.grad is not None}}


class DictLoader:
    """Yields the reference's batch format; the reference Trainer calls ``next()`` on its loader."""

    def __init__(self, batches):
        self.batches, self.i = batches, 0

    def __iter__(self):
        return self

    def __next__(self):
        b = self.batches[self.i % len(self.batches)]
        self.i += 1
        return {"input_ids": b, "labels": b}


TRAIN_STEPS, ACCUM = 6, 2


def run_trainer(model, batches, trainer_cls, config_cls, scheduler_cls, create_adamw):
    """Six optimizer steps (two micro-batches each, warm-up + cosine, clipping at 0.5) through the Trainer's own step."""
    opt = create_adamw(model, lr=1e-2, weight_decay=0.1)
    sch = scheduler_cls(opt, warmup_steps=2, max_steps=TRAIN_STEPS)
    B, S = batches[0].shape
    tc = config_cls(global_batch_size=ACCUM * B * S, micro_batch_size=B, sequence_length=S, max_steps=TRAIN_STEPS,
                    dtype=torch.float32, save_interval=10 ** 9, log_interval=10 ** 9, max_grad_norm=0.5)
    tr = trainer_cls(tc, model, opt, sch, DictLoader(batches), [])
    tr.device = torch.device("cpu")
    losses = []
    for i in range(TRAIN_STEPS):
        tr.step = i + 1
        tr._train_step_with_callbacks()
        losses.append(float(tr._metrics.get("train/CE loss")))
    return losses, {k: v.detach().clone() for k, v in model.state_dict().items()}


def run_fit_with_callbacks(model, trainer_cls, config_cls, callback_base, callbacks, create_adamw, save_dir):
    """``Trainer.fit()`` for three steps on the Trainer's own synthetic batches with the stock monitor callbacks and
    a tap: returns the metric names that reach ``log_metrics`` and the order of the lifecycle hooks."""
    seen, events = {}, []

    class Tap(callback_base):
        def log_metrics(self, metrics, step, trainer=None):
            seen.update({k: type(v).__name__ for k, v in metrics.items()})

    for hook in ("pre_train", "post_train", "pre_load_batch", "pre_step", "post_train_batch", "pre_optim_step",
                 "post_step", "pre_log_metrics", "post_log_metrics", "close"):
        setattr(Tap, hook, (lambda h: lambda self, *a, **k: events.append(h))(hook))
    opt = create_adamw(model, lr=1e-2)
    tc = config_cls(global_batch_size=2 * 32, micro_batch_size=2, sequence_length=32, max_steps=3, dtype=torch.float32,
                    save_interval=10 ** 9, log_interval=1, max_grad_norm=1.0, save_dir=save_dir)
    tr = trainer_cls(tc, model, opt, None, None, [cb() for cb in callbacks] + [Tap()])
    tr.device = torch.device("cpu")
    import contextlib
    import io

    with contextlib.redirect_stdout(io.StringIO()):
        tr.fit()
    return sorted(seen), events


def run_moe_sequence(moe_module, state_dict=None, bias_gamma=None, sign=None, steps=8):
    """Eight training forwards of one MoE layer with capacity 1.0 and adaptive capacity: outputs, drop statistics, the
    adapted capacity factor and (with ``bias_gamma``) the router's score bias after each ``post_batch``."""
    torch.manual_seed(0)
    m = moe_module.MoEBase(d_model=32, hidden_size=64, num_experts=4, top_k=2, capacity_factor=1.0,
                           adaptive_capacity=True, bias_gamma=bias_gamma)
    if sign is not None:
        m.router.config.bias_update_sign = sign
    if state_dict is not None:
        m.load_state_dict(state_dict)
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    g = torch.Generator().manual_seed(1)
    m.train()
    rows = []
    for _ in range(steps):
        x = torch.randn(2, 16, 32, generator=g)
        y = m(x)
        m.router.post_batch()
        rows.append(dict(y=y.detach().clone(), per_expert=[int(v) for v in m.per_expert_drops.tolist()],
                         capacity_factor=float(m.capacity_factor), ema=float(m.adaptive_drop_rate_ema),
                         routed=int(m.total_tokens_routed), aux=float(m.aux_loss.detach()),
                         bias=None if m.router.score_bias is None else m.router.score_bias.detach().clone()))
    return sd, rows


ATTENTION_CASES = {"bias": dict(bias=True), "qk_norm": dict(qk_norm=True), "mha": dict(n_kv_heads=None),
                   "output_dropout": dict(output_dropout=0.5),
                   "scaled_rope": dict(rope_scaling=dict(factor=4.0, original_max_position_embeddings=16))}


def run_attention(attention_cls, scaling_cls, state_dicts=None):
    """The attention module alone: causal, bidirectional and with an explicit boolean mask."""
    g = torch.Generator().manual_seed(0)
    x = torch.randn(2, 12, 64, generator=g)
    mask = (torch.rand(12, 12, generator=g) > 0.3) | torch.eye(12, dtype=torch.bool)
    out, sds = {}, {}
    for name, kw in ATTENTION_CASES.items():
        kw = dict(kw)
        if "rope_scaling" in kw:
            kw["rope_scaling"] = scaling_cls(**kw["rope_scaling"])
        torch.manual_seed(1)
        a = attention_cls(**dict(dict(d_model=64, n_heads=4, n_kv_heads=2, max_seq_len=64), **kw))
        if state_dicts is not None:
            a.load_state_dict(state_dicts[name])
        sds[name] = {k: v.detach().clone() for k, v in a.state_dict().items()}
        a.train()
        calls = {}
        for call, kw2 in (("causal", {}), ("bidirectional", dict(causal=False)),
                          ("masked", dict(causal=False, attn_mask=mask))):
            torch.manual_seed(7)             # the dropout mask of the case that has one
            calls[call] = a(x, **kw2).detach()
        # decode step: four new positions behind a cache of eight (keys already rotated, as a cache holds them)
        n_kv = kw.get("n_kv_heads", 2) or 4
        kc, vc = torch.randn(2, 8, n_kv, 16, generator=g), torch.randn(2, 8, n_kv, 16, generator=g)
        torch.manual_seed(7)
        calls["cached"] = a(x[:, :4], causal=False, kv_cache=(kc, vc), start_pos=8).detach()
        out[name] = calls
    return out, sds


TP_BLOCK = dict(n_heads=8, n_kv_heads=4, rope_base=10000.0, max_seq_len=64, qk_norm=False, ffn_hidden=128)


def tp_rank_result(transformer_cls, full_state_dict, tp_mesh):
    """One rank of a tensor-parallel run: the full weights go in, ``apply_tp`` cuts this rank's shards; returns the
    shards, the loss and the gradients of a fixed batch."""
    torch.manual_seed(0)
    m = transformer_cls(**BASE, block=dict(TP_BLOCK))
    if full_state_dict is not None:
        m.load_state_dict(full_state_dict)
    full = {k: v.detach().clone() for k, v in m.state_dict().items()}
    m.apply_tp(tp_mesh)
    ids = torch.arange(2 * 16).reshape(2, 16) % BASE["vocab_size"]
    out = m(ids, labels=ids)
    out["loss"].backward()
    return dict(full=full, shards={k: v.detach().clone() for k, v in m.state_dict().items()},
                loss=out["loss"].detach().clone(),
                grads={n: q.grad.detach().clone() for n, q in m.named_parameters() if q.grad is not None})


def _reference_tp_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    from torch.distributed.device_mesh import init_device_mesh

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    sys.path.insert(0, REF)
    from nanopsyche.model.transformer import Transformer

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("tp",))
    torch.save(tp_rank_result(Transformer, None, mesh["tp"]), os.path.join(out_dir, f"tp_rank{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def run_reference_tp(out_dir, world=2):
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as sk:
        sk.bind(("127.0.0.1", 0))
        port = sk.getsockname()[1]
    mp.spawn(_reference_tp_worker, args=(world, port, out_dir), nprocs=world)
    return [torch.load(os.path.join(out_dir, f"tp_rank{r}.pt")) for r in range(world)]


def run_routing_replay(moe_module, state_dict=None):
    """R3 routing replay: the expert choice recorded in an evaluation pass is replayed in a training pass on
    perturbed inputs (so the training logits would choose differently); outputs, router gradient and the replayed
    indices."""
    torch.manual_seed(0)
    m = moe_module.MoEBase(d_model=32, hidden_size=64, num_experts=4, top_k=2, routing_replay=True)
    if state_dict is not None:
        m.load_state_dict(state_dict)
    sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 8, 32, generator=g)
    m.eval()
    with torch.no_grad():
        _, idx, _ = m.router(x)
    m.train()
    m.router.set_replay_mask(idx)
    x2 = (x + 0.5 * torch.randn(2, 8, 32, generator=g)).requires_grad_(True)
    w2, idx2, _ = m.router(x2)
    y = m(x2)
    y.square().sum().backward()
    out = dict(idx=idx, weights=w2.detach().clone(), idx_replayed=idx2.detach().clone(), y=y.detach().clone(),
               gate_grad=m.router.gate.weight.grad.detach().clone(), x_grad=x2.grad.detach().clone())
    m.router.clear_replay_mask()
    _, idx3, _ = m.router(x2.detach())
    out["idx_after_clear"] = idx3.detach().clone()
    return sd, out


def run_moe_options(moe_module, state_dicts=None):
    """Router jitter (seeded), L2-normalised expert weights, and the phase API
    (route -> dispatch -> local_compute -> combine -> reassemble) of a single-rank layer with capacity drops."""
    out, sds = {}, {}
    g = torch.Generator().manual_seed(4)
    x = torch.randn(2, 12, 32, generator=g)
    for name, kw, l2 in (("jitter", dict(jitter_eps=0.1), False), ("l2", {}, True),
                         ("phases", dict(capacity_factor=1.0, shared_expert=True), False)):
        torch.manual_seed(0)
        m = moe_module.MoEBase(d_model=32, hidden_size=64, num_experts=4, top_k=2, **kw)
        if l2:
            m.router.config.normalize_expert_weights = "l2"
        if state_dicts is not None:
            m.load_state_dict(state_dicts[name])
        sds[name] = {k: v.detach().clone() for k, v in m.state_dict().items()}
        m.train()
        torch.manual_seed(9)
        if name != "phases":
            out[name] = m(x).detach().clone()
            continue
        B, S, D = x.shape
        x_flat, w_flat, i_flat, aux, dropped, keep = m.route(x)
        lx, lw, li, meta = m.dispatch(x_flat, i_flat, w_flat)
        eo = m.local_compute(lx, lw, li)
        y = m.reassemble(m.combine(eo, meta, x_flat, w_flat, i_flat), dropped=dropped, keep_mask=keep, B=B, S=S, D=D)
        out[name] = dict(y=y.detach().clone(), whole=m(x).detach().clone(), kept=int(x_flat.shape[0]),
                         dropped=int(dropped), keep=None if keep is None else keep.clone(), aux=float(aux.detach()))
    return out, sds


def run_small_modules(ffn_cls, norm_cls, state_dicts=None):
    """FeedForward (biases, GeGLU) and RMSNorm (fp32 and bf16 inputs, ``full_precision`` on and off) on their own."""
    g = torch.Generator().manual_seed(6)
    x = torch.randn(3, 5, 48, generator=g)
    out, sds = {}, {}
    for name, kw in (("swiglu_bias", dict(bias=True)), ("geglu", dict(activation="gelu_tanh")),
                     ("default_hidden", {})):
        torch.manual_seed(0)
        m = ffn_cls(d_model=48, **({"hidden_size": 80} if name != "default_hidden" else {}), **kw)
        if state_dicts is not None:
            m.load_state_dict(state_dicts[name])
        sds[name] = {k: v.detach().clone() for k, v in m.state_dict().items()}
        out[name] = m(x).detach().clone()
    for name, kw, dt in (("norm_fp32", {}, torch.float32), ("norm_bf16", {}, torch.bfloat16),
                         ("norm_low_precision", dict(full_precision=False), torch.bfloat16)):
        n = norm_cls(48, eps=1e-5, **kw)
        with torch.no_grad():
            n.weight.copy_(torch.linspace(0.5, 1.5, 48))
        out[name] = n(x.to(dt)).detach().clone()
    return out, sds


def main(path):
    if not os.path.isdir(os.path.join(REF, "nanopsyche")):
        print("reference not installed")
        return 3
    sys.path.insert(0, REF)
    from nanopsyche.model import moe as ref_moe
    from nanopsyche.model import rope as ref_rope
    from nanopsyche.model.transformer import Transformer
    from nanopsyche.optim.adamw import AdamW, create_adamw
    from nanopsyche.train import scheduler as ref_sched

    from nanopsyche.train.trainer import Trainer, TrainingConfig

    res = {"models": {}, "sched": {}, "rope": {}, "adamw": {}}
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, BASE["vocab_size"], (2, 32), generator=g)
    res["ids"] = ids
    for case in MODEL_CASES:
        m = build(Transformer, ref_moe, case)
        sd = {k: v.detach().clone() for k, v in m.state_dict().items()}
        res["models"][case] = dict(run_model(m, ids), state_dict=sd)

    steps = list(range(0, 130, 3))
    res["sched"]["steps"] = steps
    res["sched"]["cosine"] = [ref_sched.cosine_with_warmup(s, 10, 100, 1e-5, 3e-4) for s in steps]
    res["sched"]["wsd"] = [ref_sched.warmup_stable_decay(s, 10, 50, 40, 1e-5, 3e-4) for s in steps]
    res["sched"]["exp"] = [ref_sched.exponential_decay(s, 10, 0.97, 1e-5, 3e-4) for s in steps]
    for name, make in (("CosineWithWarmup", lambda o: ref_sched.CosineWithWarmup(o, warmup_steps=5, max_steps=40)),
                       ("WarmupStableDecay", lambda o: ref_sched.WarmupStableDecay(o, warmup_steps=5, stable_steps=20,
                                                                                   decay_steps=15))):
        p = torch.nn.Parameter(torch.zeros(2))
        opt = torch.optim.SGD([p], lr=3e-4)
        sch = make(opt)
        lrs = []
        for _ in range(50):
            lrs.append(opt.param_groups[0]["lr"])
            opt.step()
            sch.step()
        res["sched"][name] = lrs

    for name, kw in (("plain", dict(base=10000.0)), ("theta_500k", dict(base=500000.0)),
                     ("partial", dict(base=10000.0, partial_rotary_factor=0.5)),
                     ("scaled", dict(base=500000.0, scaling=ref_rope.RoPEScalingConfig(
                         factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0, original_max_position_embeddings=64)))):
        rope = ref_rope.RotaryEmbedding(32, max_seq_len=256, **kw)
        cos, sin = rope(48, offset=7, device=torch.device("cpu"))
        x = torch.randn(2, 48, 4, 32, generator=g)
        rot = int(32 * kw.get("partial_rotary_factor", 1.0))
        y = ref_rope.apply_rotary_emb(x, cos, sin) if rot == 32 else None
        res["rope"][name] = {"cos": cos, "sin": sin, "x": x, "y": y}

    # optimizer: five steps on fixed gradients; the decay / no-decay split of create_adamw by parameter name
    m = build(Transformer, ref_moe, "moe_gate_bias")
    opt = create_adamw(m, lr=1e-2, weight_decay=0.1)
    res["adamw"]["groups"] = [sorted(n for n, p in m.named_parameters() if any(p is q for q in grp["params"]))
                              for grp in opt.param_groups]
    ws = [torch.nn.Parameter(torch.randn(7, 5, generator=g)), torch.nn.Parameter(torch.randn(11, generator=g))]
    w0 = [w.detach().clone() for w in ws]
    grads = [[torch.randn(w.shape, generator=g) for w in ws] for _ in range(5)]
    opt = AdamW([{"params": [ws[0]], "weight_decay": 0.1}, {"params": [ws[1]], "weight_decay": 0.0}], lr=1e-2,
                betas=(0.9, 0.95), eps=1e-8)
    for gs in grads:
        for w, gr in zip(ws, gs):
            w.grad = gr.clone()
        opt.step()
    res["adamw"].update(w0=w0, grads=grads, w=[w.detach().clone() for w in ws])

    m = build(Transformer, ref_moe, "dense", seed=4)
    init = {k: v.detach().clone() for k, v in m.state_dict().items()}
    batches = [torch.randint(0, BASE["vocab_size"], (2, 32), generator=g) for _ in range(TRAIN_STEPS * ACCUM)]
    losses, final = run_trainer(m, batches, Trainer, TrainingConfig, ref_sched.CosineWithWarmup, create_adamw)
    res["trainer"] = dict(init=init, batches=batches, losses=losses, final=final)

    # a checkpoint directory written by the reference's checkpointer after three optimizer steps
    from nanopsyche.checkpoint.distributed import CheckpointConfig, DistributedCheckpointer

    m = build(Transformer, ref_moe, "moe_shared_expert", seed=6)
    opt = create_adamw(m, lr=1e-2, weight_decay=0.1)
    sch = ref_sched.CosineWithWarmup(opt, warmup_steps=2, max_steps=6)
    for _ in range(3):
        m(ids, labels=ids)["loss"].backward()
        opt.step()
        sch.step()
        opt.zero_grad()
    ck_dir = os.path.join(os.path.dirname(os.path.abspath(path)), "reference_checkpoints")
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=ck_dir, pinned_memory=False))
    ck.save(m, opt, sch, 3, None, {"tokens_seen": 192})
    saved = {k: v.detach().clone() for k, v in m.state_dict().items()}
    last_epoch, lr = sch.last_epoch, opt.param_groups[0]["lr"]
    m(ids, labels=ids)["loss"].backward()      # the step after the checkpoint: what a resumed run has to reproduce
    opt.step()
    res["checkpoint"] = dict(dir=ck_dir, model=saved, last_epoch=last_epoch, lr=lr,
                             after_next_step={k: v.detach().clone() for k, v in m.state_dict().items()})

    from nanopsyche.train.callbacks import GPUMemoryMonitorCallback, SpeedMonitorCallback, StabilityMonitorCallback
    from nanopsyche.train.callbacks.base import Callback

    names, events = run_fit_with_callbacks(
        build(Transformer, ref_moe, "dense"), Trainer, TrainingConfig, Callback,
        [SpeedMonitorCallback, StabilityMonitorCallback, GPUMemoryMonitorCallback], create_adamw,
        os.path.join(os.path.dirname(os.path.abspath(path)), "fit_ckpt"))
    res["fit"] = dict(metric_names=names, events=events)

    # the fault-tolerant checkpointer's directory, written by the reference
    from nanopsyche.fault_tolerance.checkpoint import FaultTolerantCheckpointer

    ft_dir = os.path.join(os.path.dirname(os.path.abspath(path)), "reference_ft")
    ft = FaultTolerantCheckpointer(ft_dir, save_interval=2, async_save=False)
    for step in (2, 3, 4):
        ft.save(m, opt, step)                       # step 3 is off the interval and skipped
    res["ft"] = dict(dir=ft_dir, latest=ft.find_latest_checkpoint(),
                     model={k: v.detach().clone() for k, v in m.state_dict().items()})

    from nanopsyche.model.attention import Attention

    att_out, att_sd = run_attention(Attention, ref_rope.RoPEScalingConfig)
    res["attention"] = dict(out=att_out, state_dicts=att_sd)

    res["tp"] = run_reference_tp(os.path.dirname(os.path.abspath(path)))

    rr_sd, rr = run_routing_replay(ref_moe)
    res["routing_replay"] = dict(state_dict=rr_sd, out=rr)

    mo_out, mo_sd = run_moe_options(ref_moe)
    res["moe_options"] = dict(out=mo_out, state_dicts=mo_sd)

    from nanopsyche.model.feed_forward import FeedForward
    from nanopsyche.model.norm import RMSNorm

    sm_out, sm_sd = run_small_modules(FeedForward, RMSNorm)
    res["small_modules"] = dict(out=sm_out, state_dicts=sm_sd)

    sd, rows = run_moe_sequence(ref_moe)
    sd_b, rows_b = run_moe_sequence(ref_moe, bias_gamma=0.05)
    res["moe_sequence"] = dict(state_dict=sd, rows=rows, state_dict_bias=sd_b, rows_bias=rows_b)
    torch.save(res, path)
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1]))
