"""Distributed semantics on CPU (gloo, 2-4 ranks): TP = unsharded, Ulysses = ring = full causal
attention, EP(ep>1) = EP(1), PP schedules = non-PP loss/grads, mesh layouts."""
import copy

import pytest
import torch
import torch.distributed as dist
import torch.nn.functional as F

from conftest import run_distributed
from nanopysche_b200.parallel import pipeline_parallel as pp
from nanopysche_b200.parallel.mesh import ParallelDims, mesh_layout


# ------------------------------------------------------------------ mesh
def test_mesh_layout_orders_and_validation():
    assert mesh_layout(8, tp_size=2, pp_size=2) == ([2, 2, 2], ["pp", "dp", "tp"])
    assert mesh_layout(8, ep_size=8) == ([1, 1, 8], ["pp", "dp", "ep"])
    assert mesh_layout(16, tp_size=2, cp_size=2, ep_size=2) == ([1, 2, 2, 2, 2], ["pp", "dp", "ep", "cp", "tp"])
    assert mesh_layout(8, dp_shard=4, dp_replicate=2) == ([1, 2, 4], ["pp", "dp_replicate", "dp_shard"])
    with pytest.raises(ValueError):
        mesh_layout(6, tp_size=4)
    d = ParallelDims(dp_shard=-1, tp=2, pp=2).set_world_size(8)
    assert d.dp_shard == 2 and d.world_size == 8 and d.layout() == ([2, 2, 2], ["pp", "dp", "tp"])
    with pytest.raises(ValueError):
        ParallelDims(tp=0)


def _mesh_worker(rank, world):
    from nanopysche_b200.parallel import mesh as M

    m = M.build_world_mesh(tp_size=2, device_type="cpu", replace=True)
    assert m.mesh_dim_names == ("pp", "dp", "tp")
    assert M.get_tp_mesh().size() == 2 and M.get_dp_model_mesh().size() == 2 and M.get_cp_mesh() is None
    assert M.get_ep_mesh().mesh_dim_names == ("dp",)
    idx, cnt = M.data_parallel_coords()
    assert cnt == 2 and idx == rank // 2
    with pytest.raises(RuntimeError):
        M.build_world_mesh(tp_size=2, device_type="cpu")
    return True


def test_world_mesh_4_ranks():
    assert all(run_distributed(_mesh_worker, 4))


# ------------------------------------------------------------------ TP
def _tp_worker(rank, world):
    from nanopysche_b200.models import Attention, FeedForward

    torch.manual_seed(0)
    att = Attention(d_model=64, n_heads=4, n_kv_heads=2, max_seq_len=16)
    ffn = FeedForward(d_model=64, hidden_size=128)
    x = torch.randn(2, 8, 64)
    xa = x.clone().requires_grad_(True)
    ref = att(xa) + ffn(xa)
    ref.sum().backward()
    ref_gx = xa.grad.clone()
    ref_gq = att.w_q.weight.grad.clone()
    att2, ffn2 = copy.deepcopy(att), copy.deepcopy(ffn)
    for m in (att2, ffn2):
        m.zero_grad()
        m.apply_tp(dist.group.WORLD)
    assert att2.w_q.weight.shape == (32, 64) and att2.w_out.weight.shape == (64, 32)
    xb = x.clone().requires_grad_(True)
    out = att2(xb) + ffn2(xb)
    out.sum().backward()
    assert torch.allclose(out, ref, atol=1e-5)
    assert torch.allclose(xb.grad, ref_gx, atol=1e-5)  # input-side backward all-reduce present
    assert torch.allclose(att2.w_q.weight.grad, ref_gq.view(2, 32, 64)[rank], atol=1e-5)
    return True


def test_tensor_parallel_matches_unsharded():
    assert all(run_distributed(_tp_worker, 2))


def _generic_tp_worker(rank, world):
    from nanopysche_b200.models.parallel_adapter import ensure_parallel_hooks

    class Layer(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = torch.nn.Linear(16, 32), torch.nn.Linear(32, 16)

        def forward(self, x):
            return self.b(F.relu(self.a(x)))

    class Net(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = torch.nn.ModuleList([Layer(), Layer()])

        def forward(self, x):
            for l in self.layers:
                x = l(x)
            return x

    torch.manual_seed(0)
    net = Net()
    x = torch.randn(3, 16)
    ref = net(x)
    net = ensure_parallel_hooks(net)
    net.apply_tp(dist.group.WORLD)
    assert torch.allclose(net(x), ref, atol=1e-5)
    return True


def test_generic_adapter_tp():
    assert all(run_distributed(_generic_tp_worker, 2))


# ------------------------------------------------------------------ CP
def _cp_worker(rank, world, ulysses):
    from nanopysche_b200.ops.attention import attention_ref
    from nanopysche_b200.parallel.context_parallel import (RingAttention, local_positions, shard_sequence,
                                                           unshard_sequence)

    torch.manual_seed(0)
    B, S, Hq, Hkv, hd = 1, 16 * world, 4, 2, 8
    q, k, v = torch.randn(B, S, Hq, hd), torch.randn(B, S, Hkv, hd), torch.randn(B, S, Hkv, hd)
    qf, kf, vf = (t.clone().requires_grad_(True) for t in (q, k, v))
    full, _ = attention_ref(qf, kf, vf, causal=True)
    full.square().sum().backward()
    ql, kl, vl = (shard_sequence(t, world, rank).clone().requires_grad_(True) for t in (q, k, v))
    pos = local_positions(S // world, world, rank)
    c = S // (2 * world)
    assert pos[0] == rank * c and pos[-1] == (2 * world - rank) * c - 1  # true zig-zag: chunks r and 2cp-1-r
    mod = RingAttention(dist.group.WORLD, use_ulysses=ulysses, use_zigzag=True)
    out = mod(ql, kl, vl, causal=True)
    assert torch.isfinite(out).all()
    assert torch.allclose(out, shard_sequence(full.detach(), world, rank), atol=1e-5)
    out.square().sum().backward()
    assert torch.allclose(ql.grad, shard_sequence(qf.grad, world, rank), atol=1e-4)
    assert torch.allclose(kl.grad, shard_sequence(kf.grad, world, rank), atol=1e-4)
    gathered = [torch.empty_like(out) for _ in range(world)]
    dist.all_gather(gathered, out.detach())
    assert torch.allclose(unshard_sequence(gathered, world), full.detach(), atol=1e-5)
    return True


@pytest.mark.parametrize("ulysses", [False, True])
def test_context_parallel_matches_full_attention(ulysses):
    assert all(run_distributed(_cp_worker, 2, ulysses))


def test_ring_attention_4_ranks():
    assert all(run_distributed(_cp_worker, 4, False))


def _cp_model_worker(rank, world):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.context_parallel import shard_batch_for_cp

    torch.manual_seed(0)
    cfg = TransformerConfig(d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=64,
                            ffn_hidden=256, qk_norm=False)
    m = cfg.build()
    x = torch.randint(0, 64, (2, 32))
    ref = m(x, labels=x)["loss"]
    ref.backward()
    g_ref = m.blocks["0"].attention.w_q.weight.grad.clone()
    m.zero_grad()
    m.apply_cp(dist.group.WORLD)
    ids, tgt = shard_batch_for_cp(x, x, world, rank)
    out = m(ids, labels=tgt, labels_shifted=True)
    assert out["loss"].item() == pytest.approx(ref.item(), rel=1e-5)  # loss over the global token count
    out["loss"].backward()
    g = m.blocks["0"].attention.w_q.weight.grad
    dist.all_reduce(g)
    assert torch.allclose(g, g_ref, atol=1e-5)  # gradients sum over the CP group
    return True


def test_context_parallel_model_loss_and_grads():
    assert all(run_distributed(_cp_model_worker, 2))


# ------------------------------------------------------------------ EP
def _ep_worker(rank, world):
    from nanopysche_b200.models.moe import ExpertParallelConfig, MoEBase, NcclAllToAllDispatcher

    torch.manual_seed(0)
    moe = MoEBase(d_model=16, hidden_size=256, num_experts=4, top_k=2, capacity_factor=None)
    torch.manual_seed(10 + rank)
    x = torch.randn(2, 6, 16)
    xa = x.clone().requires_grad_(True)
    ref = moe(xa)
    ref.sum().backward()
    full_w1_grad = moe.w1.grad.clone()
    dist.all_reduce(full_w1_grad)  # every rank's tokens contribute to every expert
    moe._aux_loss = None  # a graph tensor from the forward above cannot be deep-copied
    ep = copy.deepcopy(moe)
    ep.zero_grad()
    ep.apply_ep(ExpertParallelConfig(ep_size=world, ep_group=dist.group.WORLD, dispatcher=NcclAllToAllDispatcher()))
    assert ep.w1.shape[0] == 4 // world * 256 and ep.num_local_experts == 4 // world
    xb = x.clone().requires_grad_(True)
    out = ep(xb)
    assert torch.allclose(out, ref, atol=1e-5)
    out.sum().backward()
    assert torch.allclose(xb.grad, xa.grad, atol=1e-5)
    H = 256
    lo = rank * (4 // world)
    assert torch.allclose(ep.w1.grad, full_w1_grad[lo * H:(lo + 4 // world) * H], atol=1e-5)
    return True


def test_expert_parallel_matches_single_rank():
    assert all(run_distributed(_ep_worker, 2))


# ------------------------------------------------------------------ PP schedules
@pytest.mark.parametrize("p,m", [(2, 4), (4, 8), (4, 4), (3, 7)])
def test_schedules_validate_and_bubbles(p, m):
    g = pp.validate_schedule(pp.GPipeSchedule(p, m).generate_schedule(), p, m)
    f = pp.validate_schedule(pp.OneForwardOneBackwardSchedule(p, m).generate_schedule(), p, m)
    z = pp.validate_schedule(pp.ZeroBubbleSchedule(p, m).generate_schedule(), p, m)
    ideal = (p - 1) / (m + p - 1)
    assert g["bubble_fraction"] == pytest.approx(ideal, abs=1e-9)
    assert f["bubble_fraction"] == pytest.approx(ideal, abs=1e-9)
    assert z["bubble_fraction"] < f["bubble_fraction"] + 1e-9
    sched = pp.OneForwardOneBackwardSchedule(p, m).generate_schedule()
    for r in range(p):
        warm = min(p - 1 - r, m)
        assert [a.type for a in sched[r][:warm]] == [pp.F] * warm
    zs = pp.ZeroBubbleSchedule(p, m).generate_schedule()
    assert sum(a.type == pp.W for a in zs[0]) == m and sum(a.type == pp.BI for a in zs[0]) == m


@pytest.mark.parametrize("p,m", [(2, 4), (4, 8)])
def test_dualpipe_schedule_is_valid_and_has_no_duplicates(p, m):
    gen = pp.DualPipeSchedule(num_stages=p, num_microbatches=m)
    s = gen.generate_schedule()
    first = lambda st: 0 if st < p else p  # noqa: E731
    last = lambda st: p - 1 if st < p else 2 * p - 1  # noqa: E731
    r = pp.validate_schedule(s, p, m, stage_first=first, stage_last=last)
    fw = [(a.microbatch, a.stage) for a in s[0] if a.type == pp.F]
    assert len(fw) == len(set(fw)) == m  # each microbatch passes rank 0 once (one of its two stages)
    assert gen.stages_of_rank(0) == [0, 2 * p - 1] and gen.rank_of_stage(2 * p - 1) == 0
    one = pp.validate_schedule(pp.OneForwardOneBackwardSchedule(p, m).generate_schedule(), p, m)
    assert r["bubble_fraction"] <= one["bubble_fraction"] + 1e-9


def test_validator_rejects_bad_schedules():
    bad = [[pp.Action(pp.B, 0, 0), pp.Action(pp.F, 0, 0)], [pp.Action(pp.F, 0, 1), pp.Action(pp.B, 0, 1)]]
    with pytest.raises(ValueError):
        pp.validate_schedule(bad, 2, 1)
    dup = [[pp.Action(pp.F, 0, 0), pp.Action(pp.F, 0, 0)]]
    with pytest.raises(ValueError):
        pp.validate_schedule(dup, 1, 1)


def test_bubble_closed_forms_and_auto_schedule():
    assert pp.compute_bubble_fraction("1f1b", 4, 8) == 3 / 8
    assert pp.compute_bubble_fraction("interleaved", 4, 8, 2) == 3 / 16
    assert pp.compute_bubble_fraction("dualpipe", 8, 16) == 3 / 16
    assert pp.compute_bubble_fraction("zb1p", 4, 8) == 3 / (3 * 11)
    assert pp.compute_bubble_fraction("zbv", 4, 8) == 0.0
    from nanopysche_b200.parallel.auto_schedule import AutoScheduleConfig, AutoScheduleGenerator, StageProfile

    g = AutoScheduleGenerator([StageProfile()] * 4, AutoScheduleConfig(num_microbatches=8, num_stages=4))
    s = g.generate()
    assert len(s) == 4 and s[3][0].type == "FWD" and 0 < g.compute_bubble_fraction() < 0.5
    assert g.validate_memory()[0] and g.compute_overlap_efficiency() == 1.0
    d = AutoScheduleGenerator([StageProfile()] * 4, AutoScheduleConfig(8, 4, dualpipe_ratio=0.5))
    assert d.compute_bubble_fraction() <= g.compute_bubble_fraction() + 1e-9
    fits, peak = AutoScheduleGenerator([StageProfile(mem_gb=100)] * 4, AutoScheduleConfig(8, 4)).validate_memory()
    assert not fits and peak == 400.0


def test_stage_layer_ranges():
    from nanopysche_b200.parallel.pipeline_runtime import (PipelineParallelConfig, PipelineScheduleType,
                                                           stage_layer_ranges)

    assert stage_layer_ranges(8, 4) == [(0, 2), (2, 4), (4, 6), (6, 8)]
    assert stage_layer_ranges(10, 4) == [(0, 2), (2, 5), (5, 8), (8, 10)]  # remainder goes to stages 1..
    assert stage_layer_ranges(6, 3, [1, 3]) == [(0, 1), (1, 3), (3, 6)]
    c = PipelineParallelConfig(degree=4, schedule=PipelineScheduleType.dualpipe)
    # DualPipe: four model stages, every rank holds its own and a copy of its mirror rank's
    assert c.stages_per_rank() == 2 and c.num_stages() == 4 and c.stage_ids_this_rank(1) == [1, 2]
    cv = PipelineParallelConfig(degree=4, schedule=PipelineScheduleType.zbv_zero_bubble)
    assert cv.num_stages() == 8 and cv.stage_ids_this_rank(1) == [1, 6]
    c2 = PipelineParallelConfig(degree=4, schedule=PipelineScheduleType.interleaved_1F1B)
    assert c2.stage_ids_this_rank(1) == [1, 5]


def _pp_worker(rank, world, schedule):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.pipeline_runtime import (PipelineParallelConfig, PipelineSchedule,
                                                           PipelineScheduleType, split_model)

    torch.manual_seed(0)
    cfg = TransformerConfig(d_model=32, n_layers=4, n_heads=2, vocab_size=64, max_seq_len=16, ffn_hidden=256,
                            qk_norm=False)
    model = cfg.build()
    x = torch.randint(0, 64, (4, 8))
    ref = model(x, labels=x)["loss"]  # mean over 4 sequences = mean of the per-microbatch means here
    ref.backward()
    g_first = model.blocks["0"].attention.w_q.weight.grad.clone()
    g_last = model.blocks["3"].attention.w_q.weight.grad.clone()
    model.zero_grad()
    pcfg = PipelineParallelConfig(degree=world, schedule=PipelineScheduleType(schedule), num_microbatches=4)
    if schedule == "1F1B":      # the reference's keyword form returns its pair (stages, model chunks)
        stages, chunks = split_model(model, pp_config=pcfg, pp_rank=rank, device=torch.device("cpu"),
                                     pp_group=dist.group.WORLD)
        assert len(chunks) == len(stages) and all(a is b for a, b in zip(stages, chunks))
    else:
        stages = split_model(model, dist.group.WORLD, pcfg)
    sched = PipelineSchedule(stages, dist.group.WORLD, pcfg, hidden_shape=(1, 8, 32), hidden_dtype=torch.float32)
    loss = sched.step(x, target=x)
    def block(idx):
        for st in stages:
            if str(idx) in st.blocks:
                return st.blocks[str(idx)]
        return None

    owns_last = block(3) is not None
    assert (loss is not None) == owns_last
    if owns_last:
        assert loss.item() == pytest.approx(ref.item(), rel=1e-5)
        assert torch.allclose(block(3).attention.w_q.weight.grad, g_last, atol=1e-5)
        assert stages[-1].embeddings is None and stages[-1].lm_head is not None
    if rank == 0:
        assert stages[0].lm_head is None and stages[0].embeddings is not None
        assert torch.allclose(block(0).attention.w_q.weight.grad, g_first, atol=1e-5)
    return True


def _pp_worker_all(rank, world, schedules):
    from nanopysche_b200.ops import gemm as gemm_ops

    for sch in schedules:      # one pair of ranks for all schedules: spawning costs more than a schedule's step
        try:
            assert _pp_worker(rank, world, sch)
        except AssertionError as e:
            raise AssertionError(f"schedule {sch}: {e}") from e
        gemm_ops.SPLIT_MODE = False
        dist.barrier()
    return True


def test_pipeline_runtime_matches_single_process():
    schedules = ["1F1B", "GPipe", "InterleavedZeroBubble", "Interleaved1F1B", "ZBVZeroBubble", "LoopedBFS"]
    assert all(run_distributed(_pp_worker_all, 2, schedules, timeout=600))


def _fsdp_worker(rank, world):
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.mesh import build_world_mesh, get_dp_model_mesh

    torch.manual_seed(0)
    cfg = TransformerConfig(d_model=32, n_layers=2, n_heads=2, vocab_size=64, max_seq_len=16, ffn_hidden=256,
                            qk_norm=False)
    m = cfg.build()
    x = torch.randint(0, 64, (2, 8))
    ref = m(x, labels=x)["loss"].item()
    mesh = build_world_mesh(device_type="cpu", replace=True)
    m.apply_fsdp(get_dp_model_mesh(mesh), param_dtype=torch.float32)
    out = m(x, labels=x)
    assert out["loss"].item() == pytest.approx(ref, rel=1e-5)
    out["loss"].backward()
    assert m._fsdp_enabled
    return True


def test_fsdp_matches_unsharded_loss():
    assert all(run_distributed(_fsdp_worker, 2))


def test_nvls_allocation_is_opt_in(monkeypatch):
    """The multicast (NVLS) arenas are only asked for with NPB200_NVLS=1; otherwise the data-parallel step keeps the
    peer-load kernels and nothing is allocated."""
    import torch

    from nanopysche_b200.parallel.symm import nvls_alloc

    monkeypatch.delenv("NPB200_NVLS", raising=False)
    assert nvls_alloc(1024, torch.float32, object(), torch.device("cpu")) is None
    monkeypatch.setenv("NPB200_NVLS", "1")
    assert nvls_alloc(1024, torch.float32, None, torch.device("cpu")) is None   # no group: nothing to share with


def _tp_dp_arena_worker(rank, world):
    """tp 2 x dp 2 through parallelize_model + prepare_training's group choice: after one clipped AdamW step every
    rank's shards equal the matching slices of an unsharded model stepped on the whole batch."""
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.optim.arena import ArenaAdamW, ParamArena
    from nanopysche_b200.parallel.fsdp import DataParallelConfig
    from nanopysche_b200.parallel.mesh import build_world_mesh
    from nanopysche_b200.parallel.tensor_parallel import TensorParallelConfig
    from nanopysche_b200.parallelize import parallelize_model

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=64, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=64,
                            max_seq_len=16, qk_norm=False)
    full = cfg.build()
    model = copy.deepcopy(full)
    mesh = build_world_mesh(tp_size=2, device_type="cpu", replace=True)
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"), tp_config=TensorParallelConfig(2),
                              dp_config=DataParallelConfig(backend="arena"))
    grp = model._replica_group
    assert grp is not None and dist.get_world_size(grp) == 2
    assert getattr(model.blocks["0"].attention.w_q.weight, "_tp_sharded", None) is not None
    tp_rank, dp_rank = rank % 2, rank // 2
    torch.manual_seed(1)
    ids = torch.randint(0, 64, (4, 16))
    mine = ids[dp_rank * 2:(dp_rank + 1) * 2]
    arena = ParamArena(model, dp_group=grp, device=torch.device("cpu"))
    opt = ArenaAdamW(arena, lr=1e-2, weight_decay=0.1, max_grad_norm=0.05)
    out = model(mine, labels=mine)
    out["loss"].backward()
    opt.step()
    # oracle: the unsharded model on the whole batch (one rank, same optimizer code path)
    a0 = ParamArena(full, device=torch.device("cpu"))
    o0 = ArenaAdamW(a0, lr=1e-2, weight_decay=0.1, max_grad_norm=0.05)
    full(ids, labels=ids)["loss"].backward()
    o0.step()
    assert abs(float(opt.last_grad_norm) - float(o0.last_grad_norm)) < 1e-4 * float(o0.last_grad_norm) + 1e-6, \
        (float(opt.last_grad_norm), float(o0.last_grad_norm))
    ref = dict(full.named_parameters())
    for name, p in model.named_parameters():
        r = ref[name]
        if name.endswith(("w_q.weight", "w_k.weight", "w_v.weight", "w1.weight", "w3.weight")):
            n = r.shape[0] // 2
            r = r[tp_rank * n:(tp_rank + 1) * n]
        elif name.endswith(("w_out.weight", "w2.weight")):
            n = r.shape[1] // 2
            r = r[:, tp_rank * n:(tp_rank + 1) * n]
        assert torch.allclose(p, r, atol=2e-5, rtol=1e-4), (name, (p - r).abs().max())
    return True


def test_arena_step_with_tensor_parallel_and_data_parallel():
    assert all(run_distributed(_tp_dp_arena_worker, 4))


def _ddp_worker(rank, world):
    from nanopysche_b200.parallel.ddp import BucketedGradReducer

    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 4))
    ref = copy.deepcopy(net)
    red = BucketedGradReducer(net.parameters(), group=dist.group.WORLD, bucket_bytes=300)   # several buckets
    assert len(red.buckets) >= 2
    torch.manual_seed(5)
    x = torch.randn(4 * world, 8)
    for step in range(2):   # buckets are reusable
        net.zero_grad()
        ref.zero_grad()
        net(x[rank * 4:(rank + 1) * 4]).pow(2).mean().backward()
        red.finish()
        ref(x).pow(2).mean().backward()
        for a, b in zip(net.parameters(), ref.parameters()):
            assert torch.allclose(a.grad, b.grad, atol=1e-6), (a.grad - b.grad).abs().max()
    return True


def test_bucketed_grad_reducer_matches_full_batch():
    assert all(run_distributed(_ddp_worker, 2))


def _hsdp_worker(rank, world, backend):
    """dp_replicate 2 x dp_shard 2 on four ranks, both back ends: PyTorch FSDP2 over the 2-D mesh and the parameter
    arena (shard over dp_shard, sum over dp_replicate). One step equals the unsharded model on the whole batch."""
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.optim.arena import ArenaAdamW, ParamArena
    from nanopysche_b200.parallel.fsdp import DataParallelConfig, DataParallelType
    from nanopysche_b200.parallel.mesh import ParallelDims
    from nanopysche_b200.parallelize import parallelize_model

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=64, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=64,
                            max_seq_len=16, qk_norm=False)
    full = cfg.build()
    model = copy.deepcopy(full)
    dims = ParallelDims(dp_shard=2, dp_replicate=2)
    mesh = dims.build_mesh("cpu")
    assert tuple(mesh.mesh_dim_names) == ("pp", "dp_replicate", "dp_shard")
    torch.manual_seed(1)
    ids = torch.randint(0, 64, (8, 16))
    mine = ids[rank * 2:(rank + 1) * 2]
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"),
                              dp_config=DataParallelConfig(name=DataParallelType.hsdp, backend=backend))
    if backend == "torch":
        assert model._fsdp_enabled
        loss = model(mine, labels=mine)["loss"]
        loss.backward()
        ref_loss = full(ids, labels=ids)["loss"]
        ref_loss.backward()
        tot = loss.detach().clone()
        dist.all_reduce(tot)
        assert abs(tot.item() / world - ref_loss.item()) < 1e-5
        g = model.blocks["0"].attention.w_q.weight.grad.full_tensor()   # sharded over dp_shard, averaged over all
        assert torch.allclose(g, full.blocks["0"].attention.w_q.weight.grad, atol=1e-5)
        return True
    assert model._replicate_group is not None and dist.get_world_size(model._replica_group) == 2
    arena = ParamArena(model, dp_group=model._replica_group, replicate_group=model._replicate_group,
                       device=torch.device("cpu"))
    opt = ArenaAdamW(arena, lr=1e-2, max_grad_norm=0.05)
    model(mine, labels=mine)["loss"].backward()
    opt.step()
    a0 = ParamArena(full, device=torch.device("cpu"))
    o0 = ArenaAdamW(a0, lr=1e-2, max_grad_norm=0.05)
    full(ids, labels=ids)["loss"].backward()
    o0.step()
    assert abs(float(opt.last_grad_norm) - float(o0.last_grad_norm)) < 1e-4 * float(o0.last_grad_norm) + 1e-6
    for (n, p), q in zip(model.named_parameters(), full.parameters()):
        assert torch.allclose(p, q, atol=2e-5, rtol=1e-4), n
    return True


def _hsdp_both(rank, world):
    for backend in ("torch", "arena"):
        assert _hsdp_worker(rank, world, backend), backend
        dist.barrier()
    return True


def test_hybrid_sharded_data_parallel_four_ranks():
    assert all(run_distributed(_hsdp_both, 4, timeout=600))


def _seq_parallel_worker(rank, world):
    """Megatron sequence parallelism through library collectives (the layout of the fused TP kernels): loss and
    gradients of sharded, replicated-but-partial (norms, embeddings) and replicated (LM head) parameters match the
    unsharded model."""
    from nanopysche_b200.config import TransformerConfig

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=96, d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=64,
                            max_seq_len=16, qk_norm=False)
    model = cfg.build()
    ref = copy.deepcopy(model)
    model.apply_tp(dist.group.WORLD, sequence_parallel=True)
    assert model._tp_fused and model._tp_host
    ids = torch.randint(0, 96, (2, 16))
    dist.broadcast(ids, 0)
    for _ in range(2):      # twice: the runtime is built on the first call and reused
        model.zero_grad()
        ref.zero_grad()
        out = model(ids, labels=ids)
        out["loss"].backward()
        outr = ref(ids, labels=ids)
        outr["loss"].backward()
    assert type(model._tp_rt).__name__ == "HostTPRuntime"
    assert abs(out["loss"].item() - outr["loss"].item()) < 1e-5
    rp = dict(ref.named_parameters())
    att = model.blocks["0"].attention
    gq = rp["blocks.0.attention.w_q.weight"].grad.view(world, -1, 32)[rank]
    assert torch.allclose(att.w_q.weight.grad, gq, atol=1e-5)
    go = rp["blocks.1.attention.w_out.weight"].grad
    n_in = go.shape[1] // world
    assert torch.allclose(model.blocks["1"].attention.w_out.weight.grad, go[:, rank * n_in:(rank + 1) * n_in], atol=1e-5)
    gw2 = rp["blocks.0.feed_forward.w2.weight"].grad
    nf = gw2.shape[1] // world
    assert torch.allclose(model.blocks["0"].feed_forward.w2.weight.grad, gw2[:, rank * nf:(rank + 1) * nf], atol=1e-5)
    for name in ("blocks.0.attention_norm.weight", "blocks.1.feed_forward_norm.weight", "embeddings.weight",
                 "lm_head.weight"):
        assert torch.allclose(dict(model.named_parameters())[name].grad, rp[name].grad, atol=1e-5), name
    return True


def test_sequence_parallel_through_collectives_matches_unsharded():
    assert all(run_distributed(_seq_parallel_worker, 2))


def _seq_parallel_moe_worker(rank, world):
    """A MoE layer under sequence-parallel tensor parallelism: every TP rank routes its own rows, the load-balancing
    loss uses the statistics of all rows, and expert, router and norm gradients (all partial) are summed over the group.
    Loss, auxiliary loss and every gradient of the MoE block match the unsharded model."""
    from nanopysche_b200.config import TransformerConfig

    torch.manual_seed(0)
    cfg = TransformerConfig(d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=16,
                            ffn_hidden=64, qk_norm=False, use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2,
                            moe_offset=1, moe_hidden=32, moe_capacity_factor=None, moe_z_loss=1e-3)
    model = cfg.build()
    ref = copy.deepcopy(model)
    model.apply_tp(dist.group.WORLD, sequence_parallel=True)
    ids = torch.randint(0, 64, (2, 16))
    dist.broadcast(ids, 0)
    for _ in range(2):     # two backward passes: the partial-gradient hooks must add increments, not re-sum .grad
        out = model(ids, labels=ids)
        (out["loss"] + out["aux_loss"]).backward()
        outr = ref(ids, labels=ids)
        (outr["loss"] + outr["aux_loss"]).backward()
    assert abs(out["loss"].item() - outr["loss"].item()) < 1e-5
    assert abs(out["aux_loss"].item() - outr["aux_loss"].item()) < 1e-5
    rp = dict(ref.named_parameters())
    checked = 0
    for n, p in model.named_parameters():
        if "blocks.1" in n and p.grad is not None and p.grad.shape == rp[n].grad.shape:
            assert torch.allclose(p.grad, rp[n].grad, atol=2e-5, rtol=1e-4), n
            checked += 1
    assert checked >= 6
    return True


def test_moe_under_sequence_parallel_matches_unsharded():
    assert all(run_distributed(_seq_parallel_moe_worker, 2))


def test_reference_call_forms_of_the_pipeline_and_mesh_api():
    """The argument orders and keyword names of the reference are accepted next to this package's own."""
    import torch.nn as nn

    from nanopysche_b200.models.moe import ExpertParallelConfig, TokenDispatcher
    from nanopysche_b200.parallel.pipeline_runtime import PipelineParallelConfig as RtCfg
    from nanopysche_b200.parallel.pipeline_runtime import clip_grad_norm_pp

    stages = [nn.Linear(2, 2) for _ in range(4)]
    assert pp.GPipeSchedule(stages, 8).num_stages == 4 and pp.GPipeSchedule(4, 8).num_stages == 4
    assert pp.OneForwardOneBackwardSchedule(stages=stages, num_microbatches=8).num_stages == 4
    st = pp.PipelineStage(1, 4, nn.ModuleList([nn.Linear(2, 2)]), loss_fn=None)       # reference order
    assert st.stage_id == 1 and st.num_stages == 4 and isinstance(st.layers, nn.ModuleList)
    st = pp.PipelineStage(nn.ModuleList([nn.Linear(2, 2)]), 3, 4)
    assert st.stage_id == 3 and st.is_last
    assert RtCfg(4, schedule="1F1B").stage_ids_this_rank(2, 4) == [2]

    parts = [nn.Linear(3, 3), nn.Linear(3, 3)]
    for m in parts:
        for q in m.parameters():
            q.grad = torch.ones_like(q)
    total = clip_grad_norm_pp(parts, None, 1.0)                  # (model_parts, pp_group, max_grad_norm)
    assert total.item() == pytest.approx((2 * 12) ** 0.5)
    assert sum(q.grad.pow(2).sum() for m in parts for q in m.parameters()).sqrt().item() == pytest.approx(1.0, rel=1e-4)

    class RefStyle(TokenDispatcher):                              # a dispatcher written against the reference's ABC
        def dispatch(self, x, expert_indices, expert_weights, num_experts, ep_size, ep_rank, ep_group):
            return x, expert_weights, expert_indices, ("meta", ep_size, ep_rank)

        def combine(self, expert_output, combine_metadata, x, expert_weights, expert_indices, ep_size, ep_group):
            return expert_output + ep_size

    ep = ExpertParallelConfig(ep_size=1, dispatcher=RefStyle())
    x = torch.zeros(2, 3)
    out = ep.dispatch(x, torch.zeros(2, 1, dtype=torch.long), torch.ones(2, 1), 4)
    assert out[3] == ("meta", 1, 0) and ep.ep_rank == 0 and ep.ep_rank() == 0
    assert torch.equal(ep.combine(x, out[3], x, out[1], out[2]), x + 1)


def _seq_parallel_arena_worker(rank, world):
    """Sequence-parallel TP (tp 2) of a MoE model with the parameter arena: the MoE weights' gradients reach the arena
    past the autograd hooks' reduction (the hook leaves arena-managed parameters alone) and are summed over the TP
    group by the arena step; after one clipped AdamW step every parameter (or shard) equals the unsharded model's."""
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.optim.arena import ArenaAdamW, ParamArena
    from nanopysche_b200.parallel.mesh import build_world_mesh
    from nanopysche_b200.parallel.tensor_parallel import TensorParallelConfig
    from nanopysche_b200.parallelize import parallelize_model

    torch.manual_seed(0)
    cfg = TransformerConfig(d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=16,
                            ffn_hidden=64, qk_norm=False, use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2,
                            moe_offset=1, moe_hidden=32, moe_capacity_factor=None)
    full = cfg.build()
    model = copy.deepcopy(full)
    mesh = build_world_mesh(tp_size=2, device_type="cpu", replace=True)
    model = parallelize_model(model, world_mesh=mesh, device=torch.device("cpu"),
                              tp_config=TensorParallelConfig(2, sequence_parallel=True))
    assert model._tp_sequence_parallel and not model._tp_async
    ids = torch.randint(0, 64, (2, 16))
    dist.broadcast(ids, 0)
    arena = ParamArena(model, dp_group=None, device=torch.device("cpu"))
    assert any(r.sp_group is not None for r in arena.regions.values())
    opt = ArenaAdamW(arena, lr=1e-2, weight_decay=0.1, max_grad_norm=0.05)
    out = model(ids, labels=ids)
    (out["loss"] + out["aux_loss"]).backward()
    opt.step()
    a0 = ParamArena(full, device=torch.device("cpu"))
    o0 = ArenaAdamW(a0, lr=1e-2, weight_decay=0.1, max_grad_norm=0.05)
    o = full(ids, labels=ids)
    (o["loss"] + o["aux_loss"]).backward()
    o0.step()
    assert abs(float(opt.last_grad_norm) - float(o0.last_grad_norm)) < 1e-4 * float(o0.last_grad_norm) + 1e-6, \
        (float(opt.last_grad_norm), float(o0.last_grad_norm))
    ref = dict(full.named_parameters())
    for name, p in model.named_parameters():
        r = ref[name]
        if name.endswith(("w_q.weight", "w_k.weight", "w_v.weight", "w1.weight", "w3.weight")):
            n = r.shape[0] // 2
            r = r[rank * n:(rank + 1) * n]
        elif name.endswith(("w_out.weight", "w2.weight")):
            n = r.shape[1] // 2
            r = r[:, rank * n:(rank + 1) * n]
        assert torch.allclose(p, r, atol=2e-5, rtol=1e-4), (name, (p - r).abs().max())
    return True


def test_arena_step_under_sequence_parallel_with_moe():
    assert all(run_distributed(_seq_parallel_arena_worker, 2))


def _cp_moe_worker(rank, world):
    """Context parallelism over a MoE model: every rank routes its share of each sequence; the load-balancing loss takes
    its statistics over the whole sequence, so loss, auxiliary loss and all gradients (summed over the CP group) equal
    the single-process model's. (With per-rank statistics every rank would add a full auxiliary loss and the router's
    gradient would come out cp times too large.)"""
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.parallel.context_parallel import shard_batch_for_cp

    torch.manual_seed(0)
    cfg = TransformerConfig(d_model=32, n_layers=2, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=64,
                            ffn_hidden=64, qk_norm=False, use_moe=True, num_experts=4, moe_top_k=2, moe_interval=2,
                            moe_offset=1, moe_hidden=32, moe_capacity_factor=None, moe_z_loss=1e-3)
    m = cfg.build()
    ref = copy.deepcopy(m)
    x = torch.randint(0, 64, (2, 32))
    dist.broadcast(x, 0)
    o = ref(x, labels=x)
    (o["loss"] + o["aux_loss"]).backward()
    m.apply_cp(dist.group.WORLD)
    ids, tgt = shard_batch_for_cp(x, x, world, rank)
    out = m(ids, labels=tgt, labels_shifted=True)
    (out["loss"] + out["aux_loss"]).backward()
    assert out["loss"].item() == pytest.approx(o["loss"].item(), rel=1e-5)
    assert out["aux_loss"].item() == pytest.approx(o["aux_loss"].item(), rel=1e-5)
    rp = dict(ref.named_parameters())
    for n, p in m.named_parameters():
        if p.grad is None:
            continue
        g = p.grad.clone()
        dist.all_reduce(g)
        assert torch.allclose(g, rp[n].grad, atol=2e-5, rtol=1e-4), n
    return True


def test_context_parallel_with_moe_matches_single_process():
    assert all(run_distributed(_cp_moe_worker, 2))
