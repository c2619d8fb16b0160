"""Compositions of the parallel dimensions through ``parallelize_model`` + ``Trainer`` on gloo ranks: one SGD step with
learning rate 1 and no clipping turns every parameter's change into the gradient the framework applied, which must equal
the gradient of the single-process model under the data-parallel objective (the mean over the ranks that read
different batches of each rank's cross-entropy plus auxiliary loss) - for replicated parameters, tensor-parallel
shards, expert shards and parameters applied to row shards alike."""
import copy
import os

import pytest
import torch
import torch.distributed as dist

from conftest import run_distributed


def _worker(rank, world, dims, moe, seq_par):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.context_parallel import ContextParallelConfig
    from nanopysche_b200.parallel.mesh import build_world_mesh, data_parallel_coords
    from nanopysche_b200.parallel.tensor_parallel import TensorParallelConfig
    from nanopysche_b200.parallelize import parallelize_model
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig

    torch.manual_seed(0)
    kw = dict(use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2, moe_offset=1, moe_hidden=32,
              moe_capacity_factor=None, moe_bias_gamma=1e-2) if moe else {}
    cfg = TransformerConfig(d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=32,
                            ffn_hidden=64, qk_norm=False, **kw)
    model = cfg.build()
    ref = copy.deepcopy(model)
    mesh = build_world_mesh(device_type="cpu", replace=True, **dims)
    idx, cnt = data_parallel_coords(mesh)
    torch.manual_seed(1)
    batches = [torch.randint(0, 64, (2, 16)) for _ in range(cnt)]
    for b in batches:
        o = ref(b, labels=b)
        ((o["loss"] + (o["aux_loss"] if o.get("aux_loss") is not None else 0)) / cnt).backward()
    tp, cp, ep = dims.get("tp_size", 1), dims.get("cp_size", 1), dims.get("ep_size", 1)
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"),
                              tp_config=TensorParallelConfig(tp, sequence_parallel=seq_par) if tp > 1 else None,
                              cp_config=ContextParallelConfig(cp) if cp > 1 else None)
    opt = torch.optim.SGD(model.parameters(), lr=1.0)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    mine = batches[idx]

    class Loader:
        def __iter__(self):
            return iter([(mine, mine.clone())])

    tc = TrainingConfig(global_batch_size=cnt * 2 * 16, micro_batch_size=2, sequence_length=16, max_steps=1,
                        dtype=torch.float32, log_interval=0, save_interval=0, vocab_size=64, dp_world_size=cnt,
                        max_grad_norm=0.0, cp_size=cp)
    Trainer(tc, model, opt, data_loader=Loader(), device=torch.device("cpu")).fit()
    names = mesh.mesh_dim_names
    tp_rank = mesh["tp"].get_local_rank() if "tp" in names else 0
    ep_rank = mesh["ep"].get_local_rank() if "ep" in names else 0
    rp = dict(ref.named_parameters())
    bad = {}
    for n, p in model.named_parameters():
        g, r = before[n] - p.detach(), rp[n].grad
        if tp > 1 and n.endswith(("w_q.weight", "w_k.weight", "w_v.weight", "w1.weight", "w3.weight")):
            k = r.shape[0] // tp
            r = r[tp_rank * k:(tp_rank + 1) * k]
        elif tp > 1 and n.endswith(("w_out.weight", "w2.weight")):
            k = r.shape[1] // tp
            r = r[:, tp_rank * k:(tp_rank + 1) * k]
        if getattr(p, "_ep_sharded", False):
            k = r.shape[0] // ep
            r = r[ep_rank * k:(ep_rank + 1) * k]
        err = float((g - r).abs().max() / (r.abs().max() + 1e-12)) if g.shape == r.shape else float("inf")
        if err > 2e-3:
            bad[n] = err
    _ref_bias_update(ref)
    _check_biases(model, ref, bad)
    return bad


def _ref_bias_update(ref):
    """The single-process model's DeepSeek-V3 bias update from the counts of everything it routed."""
    for m in ref.modules():
        if hasattr(m, "post_batch") and hasattr(m, "score_bias") and m.score_bias is not None:
            m.post_batch(groups=[])


def _check_biases(model, ref, bad):
    rb = {n: b for n, b in ref.named_buffers() if n.endswith("score_bias")}
    for n, b in model.named_buffers():
        if n.endswith("score_bias"):
            key = n.split(".", 2)[2] if n.startswith("stages.") else n
            key = key.replace(".module.", ".")
            if not torch.allclose(b, rb[key], atol=1e-7):
                bad[n] = ("score_bias", float((b - rb[key]).abs().max()))


def _many(rank, world, fn, cases):
    """Run several compositions inside one set of ranks (each builds its own mesh): spawning ranks costs more than a
    case does. Returns ``{case id: mismatches}`` for the cases that did not match."""
    out = {}
    for cid, args in cases:
        bad = fn(rank, world, *args)
        if bad:
            out[cid] = bad
        dist.barrier()
    return out


def _check(res):
    bad = {}
    for r in res:
        for cid, b in r.items():
            bad.setdefault(cid, {}).update(b)
    assert not bad, bad


def test_applied_gradients_match_single_process():
    cases = [("dp2xtp2sp-moe", (dict(tp_size=2), True, True)),
             ("ep2xtp2sp-moe", (dict(ep_size=2, tp_size=2), True, True)),
             ("ep2xtp2-moe", (dict(ep_size=2, tp_size=2), True, False)),
             ("cp2xep2-moe", (dict(cp_size=2, ep_size=2), True, False)),
             ("cp2xtp2sp-moe", (dict(cp_size=2, tp_size=2), True, True)),
             ("dp2xcp2-dense", (dict(cp_size=2), False, False))]
    _check(run_distributed(_many, 4, _worker, cases, timeout=600))


def _pp_worker(rank, world, dims, moe, seq_par, schedule):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.mesh import build_world_mesh, data_parallel_coords
    from nanopysche_b200.parallel.tensor_parallel import TensorParallelConfig
    from nanopysche_b200.parallel.context_parallel import ContextParallelConfig
    from nanopysche_b200.parallel.pipeline_parallel import PipelineParallelConfig
    from nanopysche_b200.parallelize import parallelize_model
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig
    torch.manual_seed(0)
    kw = dict(use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2, moe_offset=1, moe_hidden=32,
              moe_capacity_factor=None, moe_bias_gamma=1e-2) if moe else {}
    cfg = TransformerConfig(d_model=32, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=32,
                            ffn_hidden=64, qk_norm=False, **kw)
    model = cfg.build()
    ref = copy.deepcopy(model)
    mesh = build_world_mesh(device_type="cpu", replace=True, **dims)
    idx, cnt = data_parallel_coords(mesh)
    torch.manual_seed(1)
    M = 2
    batches = [torch.randint(0, 64, (4, 16)) for _ in range(cnt)]
    for b in batches:
        for mb in b.chunk(M):
            o = ref(mb, labels=mb)
            ((o["loss"] + (o["aux_loss"] if o.get("aux_loss") is not None else 0)) / (cnt * M)).backward()
    tp, cp, ep, pp = dims.get("tp_size", 1), dims.get("cp_size", 1), dims.get("ep_size", 1), dims.get("pp_size", 1)
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"),
                              pp_config=PipelineParallelConfig(pp, schedule=schedule, num_microbatches=M),
                              tp_config=TensorParallelConfig(tp, sequence_parallel=seq_par) if tp > 1 else None,
                              cp_config=ContextParallelConfig(cp) if cp > 1 else None)
    opt = torch.optim.SGD(model.parameters(), lr=1.0)
    before = {n: p.detach().clone() for n, p in model.named_parameters()}
    mine = batches[idx]
    class Loader:
        def __iter__(self):
            return iter([(mine, mine.clone())])
    tc = TrainingConfig(global_batch_size=cnt * 4 * 16, micro_batch_size=4, sequence_length=16, max_steps=1,
                        dtype=torch.float32, log_interval=0, save_interval=0, vocab_size=64, dp_world_size=cnt,
                        max_grad_norm=0.0, cp_size=cp, pp_schedule=schedule, pp_microbatches=M)
    Trainer(tc, model, opt, data_loader=Loader(), device=torch.device("cpu")).fit()
    names = mesh.mesh_dim_names
    tp_rank = mesh["tp"].get_local_rank() if "tp" in names else 0
    ep_rank = mesh["ep"].get_local_rank() if "ep" in names else 0
    rp = dict(ref.named_parameters())
    bad = {}
    for n, p in model.named_parameters():
        key = n.split(".", 2)[2] if n.startswith("stages.") else n
        if key not in rp:
            bad[n] = "missing"
            continue
        g, r = before[n] - p.detach(), rp[key].grad
        if tp > 1 and key.endswith(("w_q.weight", "w_k.weight", "w_v.weight", "w1.weight", "w3.weight")):
            k = r.shape[0] // tp
            r = r[tp_rank * k:(tp_rank + 1) * k]
        elif tp > 1 and key.endswith(("w_out.weight", "w2.weight")):
            k = r.shape[1] // tp
            r = r[:, tp_rank * k:(tp_rank + 1) * k]
        if getattr(p, "_ep_sharded", False):
            k = r.shape[0] // ep
            r = r[ep_rank * k:(ep_rank + 1) * k]
        if g.shape != r.shape:
            bad[n] = "shape"
            continue
        e = float((g - r).abs().max() / (r.abs().max() + 1e-12))
        if e > 2e-3:
            bad[n] = round(e, 4)
    _ref_bias_update(ref)
    _check_biases(model, ref, bad)
    return bad


def test_applied_gradients_match_single_process_under_pipelines():
    """The same check with a pipeline in the composition: the reference objective is the mean over micro-batches (and
    data-parallel ranks) of each micro-batch's loss, as the schedule computes it."""
    cases = [("pp2xcp2-dense-1f1b", (dict(pp_size=2, cp_size=2), False, False, "1F1B")),
             ("pp2xep2-moe-1f1b", (dict(pp_size=2, ep_size=2), True, False, "1F1B")),
             ("pp2xtp2sp-moe-dualpipe", (dict(pp_size=2, tp_size=2), True, True, "DualPipe")),
             ("pp2xep2-moe-dualpipe", (dict(pp_size=2, ep_size=2), True, False, "DualPipe"))]
    _check(run_distributed(_many, 4, _pp_worker, cases, timeout=600))


def _fsdp_worker(rank, world, dims, moe, seq_par, hsdp, clip):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.fsdp import DataParallelConfig
    from nanopysche_b200.parallel.mesh import build_world_mesh, data_parallel_coords
    from nanopysche_b200.parallel.tensor_parallel import TensorParallelConfig
    from nanopysche_b200.parallelize import parallelize_model
    from nanopysche_b200.parallel.context_parallel import ContextParallelConfig
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig
    torch.manual_seed(0)
    kw = dict(use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2, moe_offset=1, moe_hidden=32,
              moe_capacity_factor=None, moe_bias_gamma=1e-2) if moe else {}
    cfg = TransformerConfig(d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=32,
                            ffn_hidden=64, qk_norm=False, **kw)
    model = cfg.build()
    ref = copy.deepcopy(model)
    mesh = build_world_mesh(device_type="cpu", replace=True, **dims, **hsdp)
    idx, cnt = data_parallel_coords(mesh)
    torch.manual_seed(1)
    batches = [torch.randint(0, 64, (2, 16)) for _ in range(cnt)]
    for b in batches:
        o = ref(b, labels=b)
        ((o["loss"] + (o["aux_loss"] if o.get("aux_loss") is not None else 0)) / cnt).backward()
    tp, ep = dims.get("tp_size", 1), dims.get("ep_size", 1)
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"),
                              tp_config=TensorParallelConfig(tp, sequence_parallel=seq_par) if tp > 1 else None,
                              cp_config=ContextParallelConfig(dims.get("cp_size", 1)) if dims.get("cp_size", 1) > 1 else None,
                              dp_config=DataParallelConfig(backend="torch", param_dtype=torch.float32))
    CLIP = clip
    if CLIP:
        torch.nn.utils.clip_grad_norm_(ref.parameters(), CLIP)
    opt = torch.optim.SGD(model.parameters(), lr=1.0)
    def full(p):
        return p.full_tensor() if hasattr(p, "full_tensor") else p
    before = {n: full(p.detach()).clone() for n, p in model.named_parameters()}
    mine = batches[idx]
    class Loader:
        def __iter__(self):
            return iter([(mine, mine.clone())])
    tc = TrainingConfig(global_batch_size=cnt * 2 * 16, micro_batch_size=2, sequence_length=16, max_steps=1,
                        dtype=torch.float32, log_interval=0, save_interval=0, vocab_size=64, dp_world_size=cnt,
                        max_grad_norm=CLIP, cp_size=dims.get("cp_size", 1))
    Trainer(tc, model, opt, data_loader=Loader(), device=torch.device("cpu")).fit()
    names = mesh.mesh_dim_names
    tp_rank = mesh["tp"].get_local_rank() if "tp" in names else 0
    ep_rank = mesh["ep"].get_local_rank() if "ep" in names else 0
    rp = dict(ref.named_parameters())
    bad = {}
    for n, p in model.named_parameters():
        g, r = before[n] - full(p.detach()), rp[n].grad
        if tp > 1 and n.endswith(("w_q.weight", "w_k.weight", "w_v.weight", "w1.weight", "w3.weight")):
            k = r.shape[0] // tp
            r = r[tp_rank * k:(tp_rank + 1) * k]
        elif tp > 1 and n.endswith(("w_out.weight", "w2.weight")):
            k = r.shape[1] // tp
            r = r[:, tp_rank * k:(tp_rank + 1) * k]
        if ".moe.w" in n and ep > 1:
            k = r.shape[0] // ep
            r = r[ep_rank * k:(ep_rank + 1) * k]
        if g.shape != r.shape:
            bad[n] = ("shape", tuple(g.shape), tuple(r.shape))
            continue
        e = float((g - r).abs().max() / (r.abs().max() + 1e-12))
        if e > 2e-3:
            bad[n] = round(e, 4)
    _ref_bias_update(ref)
    _check_biases(model, ref, bad)
    return bad


def test_applied_gradients_match_single_process_under_torch_fsdp2():
    """PyTorch FSDP2 (the reference's data-parallel mechanism) shards and averages over the dp dims only; the Trainer
    combines the gradients over the EP / CP dims afterwards and clips with one norm over TP, expert and FSDP shards.
    One clipped SGD step against the clipped single-process gradient."""
    cases = [("fsdp2xtp2", (dict(tp_size=2), False, False, {}, 0.05)),
             ("fsdp2xep2-moe", (dict(ep_size=2), True, False, {}, 0.05)),
             ("fsdp2xcp2", (dict(cp_size=2), False, False, {}, 0.05)),
             ("fsdp2xtp2sp-moe", (dict(tp_size=2), True, True, {}, 0.05)),
             ("hsdp2x2", ({}, False, False, dict(dp_replicate=2, dp_shard=2), 0.05))]
    _check(run_distributed(_many, 4, _fsdp_worker, cases, timeout=600))


def _pp_arena_worker(rank, world, dims, moe, seq_par, schedule):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.mesh import build_world_mesh, data_parallel_coords
    from nanopysche_b200.parallel.tensor_parallel import TensorParallelConfig
    from nanopysche_b200.parallel.context_parallel import ContextParallelConfig
    from nanopysche_b200.parallel.pipeline_parallel import PipelineParallelConfig
    from nanopysche_b200.parallelize import parallelize_model
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig
    torch.manual_seed(0)
    kw = dict(use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2, moe_offset=1, moe_hidden=32,
              moe_capacity_factor=None, moe_bias_gamma=1e-2) if moe else {}
    cfg = TransformerConfig(d_model=32, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=32,
                            ffn_hidden=64, qk_norm=False, **kw)
    model = cfg.build()
    ref = copy.deepcopy(model)
    mesh = build_world_mesh(device_type="cpu", replace=True, **dims)
    idx, cnt = data_parallel_coords(mesh)
    torch.manual_seed(1)
    M = 2
    batches = [torch.randint(0, 64, (4, 16)) for _ in range(cnt)]
    from nanopysche_b200.optim.arena import ArenaAdamW, ParamArena
    a0 = ParamArena(ref, device=torch.device("cpu"))
    o0 = ArenaAdamW(a0, lr=1e-2, weight_decay=0.1, max_grad_norm=0.05)
    for b in batches:
        for mb in b.chunk(M):
            o = ref(mb, labels=mb)
            ((o["loss"] + (o["aux_loss"] if o.get("aux_loss") is not None else 0)) / (cnt * M)).backward()
    o0.step()
    tp, cp, ep, pp = dims.get("tp_size", 1), dims.get("cp_size", 1), dims.get("ep_size", 1), dims.get("pp_size", 1)
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"),
                              pp_config=PipelineParallelConfig(pp, schedule=schedule, num_microbatches=M),
                              tp_config=TensorParallelConfig(tp, sequence_parallel=seq_par) if tp > 1 else None,
                              cp_config=ContextParallelConfig(cp) if cp > 1 else None)
    arena = ParamArena(model, dp_group=getattr(model, "_replica_group", None), device=torch.device("cpu"),
                       expert_replica_group=getattr(model, "_expert_replica_group", None))
    opt = ArenaAdamW(arena, lr=1e-2, weight_decay=0.1, max_grad_norm=0.05)
    opt.norm_groups = [model._pp_group]
    opt.norm_copies = 2.0 if getattr(model, "is_dualpipe", False) else 1.0
    mine = batches[idx]
    class Loader:
        def __iter__(self):
            return iter([(mine, mine.clone())])
    tc = TrainingConfig(global_batch_size=cnt * 4 * 16, micro_batch_size=4, sequence_length=16, max_steps=1,
                        dtype=torch.float32, log_interval=0, save_interval=0, vocab_size=64, dp_world_size=cnt,
                        max_grad_norm=0.05, cp_size=cp, pp_schedule=schedule, pp_microbatches=M)
    Trainer(tc, model, opt, data_loader=Loader(), device=torch.device("cpu")).fit()
    names = mesh.mesh_dim_names
    tp_rank = mesh["tp"].get_local_rank() if "tp" in names else 0
    ep_rank = mesh["ep"].get_local_rank() if "ep" in names else 0
    rp = dict(ref.named_parameters())
    bad = {}
    gn = (float(opt.last_grad_norm), float(o0.last_grad_norm))
    if abs(gn[0] - gn[1]) > 1e-3 * gn[1]:
        bad["grad_norm"] = gn
    for n, p in model.named_parameters():
        key = n.split(".", 2)[2] if n.startswith("stages.") else n
        if key not in rp:
            bad[n] = "missing"
            continue
        g, r = p.detach(), rp[key].detach()
        if tp > 1 and key.endswith(("w_q.weight", "w_k.weight", "w_v.weight", "w1.weight", "w3.weight")):
            k = r.shape[0] // tp
            r = r[tp_rank * k:(tp_rank + 1) * k]
        elif tp > 1 and key.endswith(("w_out.weight", "w2.weight")):
            k = r.shape[1] // tp
            r = r[:, tp_rank * k:(tp_rank + 1) * k]
        if getattr(p, "_ep_sharded", False):
            k = r.shape[0] // ep
            r = r[ep_rank * k:(ep_rank + 1) * k]
        if g.shape != r.shape:
            bad[n] = "shape"
            continue
        e = float((g - r).abs().max())
        if e > 5e-5:
            bad[n] = round(e, 6)
    _ref_bias_update(ref)
    _check_biases(model, ref, bad)
    return bad


def test_arena_optimizer_under_pipelines_matches_single_process():
    """The parameter arena (CPU reference path of the fused optimizer) behind pipeline schedules with deferred
    weight-gradient GEMMs: clipping norm over all stages (``norm_groups``, DualPipe's twin copies counted once) and the
    weights after one clipped AdamW step equal the single-process arena step."""
    cases = [("pp2xdp2-dense-zbv-arena", (dict(pp_size=2), False, False, "ZBVZeroBubble")),
             ("pp2xtp2sp-moe-dualpipe-arena", (dict(pp_size=2, tp_size=2), True, True, "DualPipe"))]
    _check(run_distributed(_many, 4, _pp_arena_worker, cases, timeout=600))


def _build_for_resume(dims, sp, schedule):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.mesh import build_world_mesh
    from nanopysche_b200.parallel.tensor_parallel import TensorParallelConfig
    from nanopysche_b200.parallel.pipeline_parallel import PipelineParallelConfig
    from nanopysche_b200.parallelize import parallelize_model
    torch.manual_seed(0)
    cfg = TransformerConfig(d_model=32, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=32,
                            ffn_hidden=64, qk_norm=False, use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2,
                            moe_offset=1, moe_hidden=32, moe_capacity_factor=None, moe_bias_gamma=1e-2)
    model = cfg.build()
    mesh = build_world_mesh(device_type="cpu", replace=True, **dims)
    tp, pp = dims.get("tp_size", 1), dims.get("pp_size", 1)
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"),
                              pp_config=PipelineParallelConfig(pp, schedule=schedule, num_microbatches=2) if pp > 1 else None,
                              tp_config=TensorParallelConfig(tp, sequence_parallel=sp) if tp > 1 else None)
    return model, mesh


def _resume_worker(rank, world, dims, sp, schedule, save_dir):
    from nanopysche_b200.checkpoint.distributed import CheckpointConfig, DistributedCheckpointer
    from nanopysche_b200.parallel.mesh import data_parallel_coords
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig
    def run(model, mesh, steps, ck=None, resume=False, start_batches=0):
        idx, cnt = data_parallel_coords(mesh)
        torch.manual_seed(1)
        allb = [[torch.randint(0, 64, (4, 16)) for _ in range(cnt)] for _ in range(4)]
        mine = [allb[s][idx] for s in range(4)][start_batches:]
        opt = torch.optim.AdamW(model.parameters(), lr=1e-2)
        class Loader:
            def __iter__(self):
                return iter([(b, b.clone()) for b in mine])
        tc = TrainingConfig(global_batch_size=cnt * 4 * 16, micro_batch_size=4, sequence_length=16, max_steps=steps,
                            dtype=torch.float32, log_interval=0, save_interval=0, vocab_size=64, dp_world_size=cnt,
                            max_grad_norm=1.0, pp_schedule=schedule, pp_microbatches=2, save_dir=save_dir)
        tr = Trainer(tc, model, opt, data_loader=Loader(), device=torch.device("cpu"), checkpointer=ck)
        if resume:
            tr.load_checkpoint(save_dir)
        tr.fit()
        return tr, opt
    # uninterrupted: 3 steps
    m1, mesh = _build_for_resume(dims, sp, schedule)
    run(m1, mesh, 3)
    # interrupted: 2 steps, save, rebuild, resume, 1 more step
    m2, mesh = _build_for_resume(dims, sp, schedule)
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=save_dir, pinned_memory=False))
    tr, opt = run(m2, mesh, 2, ck=ck)
    ck.save(tr.step, m2, opt)
    m3, mesh = _build_for_resume(dims, sp, schedule)
    for p in m3.parameters():
        p.data.add_(1.0)     # make sure the load does something
    ck3 = DistributedCheckpointer(CheckpointConfig(save_dir=save_dir, pinned_memory=False))
    tr3, _ = run(m3, mesh, 3, ck=ck3, resume=True, start_batches=2)
    bad = {}
    for (n, a), (_, b) in zip(m1.named_parameters(), m3.named_parameters()):
        e = float((a.detach() - b.detach()).abs().max())
        if e > 1e-5:
            bad[n] = e
    for (n, a), (_, b) in zip(m1.named_buffers(), m3.named_buffers()):
        if n.endswith("score_bias") and float((a - b).abs().max()) > 1e-6:
            bad[n] = "bias"
    assert tr3.step == 3
    return bad


def _resume_cases(rank, world, root):
    out = {}
    for cid, dims, sp, sch in (("tp2sp-x-ep2", dict(tp_size=2, ep_size=2), True, "1F1B"),
                               ("pp2-dualpipe-x-ep2", dict(pp_size=2, ep_size=2), False, "DualPipe")):
        bad = _resume_worker(rank, world, dims, sp, sch, os.path.join(root, cid))
        if bad:
            out[cid] = bad
        dist.barrier()
    return out


def test_resume_under_compositions_is_exact(tmp_path):
    """Two steps, a checkpoint, a freshly built (and deliberately perturbed) model that resumes and takes the third
    step: weights and router biases equal those of three uninterrupted steps - with tensor-parallel, expert and
    sequence-parallel shards, and with DualPipe's two stage copies per rank."""
    _check(run_distributed(_resume_cases, 4, str(tmp_path), timeout=600))
