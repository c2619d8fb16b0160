"""Trainer loop, callbacks, data, optimizers, checkpointing and fault handling (CPU; faults are
injected on the host: a stalled rank, a truncated shard, an exception inside a step)."""
import json
import os
import time

import numpy as np
import pytest
import torch

import torch.distributed as dist
from conftest import run_distributed
from nanopysche_b200.checkpoint.distributed import (CheckpointConfig, DistributedCheckpointer,
                                                    IncrementalCheckpointer, PinnedMemoryStager, PlanCache)
from nanopysche_b200.config import TransformerConfig
from nanopysche_b200.fault_tolerance import (CommTimeoutError, FaultTolerantCheckpointer, HangDetector,
                                             HeartbeatCoordinator)
from nanopysche_b200.optim import AdamW, DiLoCoCompressor, create_adamw
from nanopysche_b200.optim.arena import ArenaAdamW, ParamArena
from nanopysche_b200.train import (CosineWithWarmup, DistributedDataLoader, DistributedDataset, Trainer,
                                   create_distributed_loader)
from nanopysche_b200.train.callbacks import (Callback, ConsoleLoggerCallback, ProfilerCallback, SpeedMonitorCallback,
                                             StabilityMonitorCallback)
from nanopysche_b200.train.trainer import TrainingConfig


def tiny_model(moe=False):
    torch.manual_seed(0)
    return TransformerConfig(d_model=32, n_layers=2, n_heads=2, vocab_size=64, max_seq_len=16, ffn_hidden=256,
                             qk_norm=False, use_moe=moe, num_experts=4, moe_interval=1, moe_hidden=256).build()


class Recorder(Callback):
    def __init__(self):
        self.events, self.logged = [], []

    def pre_train(self, t): self.events.append("pre_train")
    def pre_load_batch(self, t): self.events.append("pre_load_batch")
    def pre_step(self, t, b): self.events.append("pre_step")
    def post_train_batch(self, t): self.events.append("post_train_batch")
    def pre_optim_step(self, t): self.events.append("pre_optim_step")
    def post_step(self, t): self.events.append("post_step")
    def log_metrics(self, m, s, t): self.logged.append((s, dict(m)))
    def post_train(self, t): self.events.append("post_train")
    def on_error(self, t, e): self.events.append("on_error")
    def close(self, t): self.events.append("close")


def test_trainer_trains_and_calls_every_hook(tmp_path):
    m = tiny_model(moe=True)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-3)
    tokens = np.random.RandomState(0).randint(0, 64, size=4000).astype(np.uint16)
    loader = create_distributed_loader(tokens, 2, 16, shuffle=False)
    rec = Recorder()
    tc = TrainingConfig(global_batch_size=2 * 16 * 2, micro_batch_size=2, sequence_length=16, max_steps=6,
                        log_interval=2, save_interval=0, dtype=torch.float32, vocab_size=64)
    assert tc.gradient_accumulation_steps == 2
    tr = Trainer(tc, m, opt, CosineWithWarmup(opt, 1, 6), loader,
                 [rec, SpeedMonitorCallback(), StabilityMonitorCallback(), ConsoleLoggerCallback()])
    tr.fit()
    assert tr.step == 6 and tr.tokens_seen == 6 * 64
    assert rec.events[0] == "pre_train" and rec.events[-2:] == ["post_train", "close"]
    assert rec.events[1:7] == ["pre_load_batch", "pre_step", "post_train_batch", "pre_optim_step", "post_step",
                               "pre_load_batch"]
    steps = [s for s, _ in rec.logged]
    assert steps == [2, 4, 6]
    last = rec.logged[-1][1]
    for k in ("train/CE loss", "train/PPL", "optim/LR", "optim/total grad norm", "throughput/total tokens",
              "throughput/device/TPS", "throughput/device/MFU", "spike/SpikeScore", "throughput/step_time (s)"):
        assert k in last, k
    assert rec.logged[-1][1]["train/CE loss"] < rec.logged[0][1]["train/CE loss"]


def test_trainer_synthetic_batches_and_error_hook():
    m = tiny_model()
    opt = torch.optim.SGD(m.parameters(), lr=0.1)
    rec = Recorder()

    class Boom(Callback):
        def post_train_batch(self, t):
            if t.step == 1:
                raise RuntimeError("injected failure")

    tc = TrainingConfig(global_batch_size=32, micro_batch_size=2, sequence_length=16, max_steps=4, log_interval=1,
                        save_interval=0, dtype=torch.float32, vocab_size=64)
    tr = Trainer(tc, m, opt, None, None, [rec, Boom()])
    with pytest.raises(RuntimeError, match="injected"):
        tr.fit()
    assert "on_error" in rec.events and rec.events[-1] == "close" and tr.step == 1


def test_trainer_raises_comm_timeout_from_the_device_status_word(tmp_path):
    """A stubbed status reader stands in for a kernel whose bounded wait ran out (code 2: flag wait): the trainer
    sees it at the next metric flush, raises CommTimeoutError, runs on_error and writes an emergency checkpoint."""
    from nanopysche_b200.fault_tolerance.hang_detection import CommTimeoutError

    m = tiny_model()
    opt = torch.optim.SGD(m.parameters(), lr=0.1)
    rec = Recorder()
    calls = {"n": 0}

    def reader():
        calls["n"] += 1
        return (2, 11, 3, 250, 0, 0, 0, 0) if calls["n"] >= 3 else (0,) * 8

    tc = TrainingConfig(global_batch_size=32, micro_batch_size=2, sequence_length=16, max_steps=8, log_interval=1,
                        save_interval=0, save_dir=str(tmp_path), dtype=torch.float32, vocab_size=64)
    tr = Trainer(tc, m, opt, None, None, [rec], status_reader=reader)
    with pytest.raises(CommTimeoutError, match="flag wait timed out"):
        tr.fit()
    assert tr.step == 3 and "on_error" in rec.events and rec.events[-1] == "close"
    d = tr.emergency_checkpoint_dir
    assert d is not None and os.path.isfile(os.path.join(d, "rank_0000_model.pt"))
    sd = torch.load(os.path.join(d, "rank_0000_model.pt"), weights_only=False)
    assert torch.equal(sd["lm_head.weight"], m.lm_head.weight.detach())


def test_dataset_and_loader_iterator_protocol():
    tokens = np.arange(1000, dtype=np.uint16)
    ds = DistributedDataset(tokens, 10)
    ids, labels = ds[3]
    assert len(ds) == 99 and ids.tolist() == list(range(30, 40)) and torch.equal(ids, labels)
    dl = DistributedDataLoader(ds, 4, shuffle=False, dp_rank=1, dp_world=2)
    first = next(dl)
    a, _ = first
    assert a.shape == (4, 10) and a[0, 0].item() == 10  # rank 1 of 2 takes odd samples
    # the reference's mapping access on samples and collated batches alike
    assert first["input_ids"] is a and torch.equal(first["labels"], first.labels) and "labels" in first
    assert first.keys() == ["input_ids", "labels"] and first.get("attention_mask") is None
    assert torch.equal(ds[3]["input_ids"], ids) and dict(ds[3].items())["labels"] is not None
    n = len(dl)
    for _ in range(n + 2):  # runs past the end of an epoch without StopIteration
        next(dl)
    assert dl.epoch == 1 and dl.state_dict()["batches_served"] == n + 3


def test_adamw_matches_torch_and_param_groups():
    torch.manual_seed(0)
    w1 = torch.nn.Parameter(torch.randn(8, 8))
    w2 = torch.nn.Parameter(w1.detach().clone())
    a = AdamW([w1], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1)
    b = torch.optim.AdamW([w2], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    for _ in range(5):
        g = torch.randn(8, 8)
        w1.grad, w2.grad = g.clone(), g.clone()
        a.step()
        b.step()
    assert torch.allclose(w1, w2, atol=1e-6)
    opt = create_adamw(tiny_model())
    decay, no_decay = opt.param_groups
    assert decay["weight_decay"] == 0.1 and no_decay["weight_decay"] == 0.0
    assert all(p.dim() >= 2 for p in decay["params"]) and any(p.dim() == 1 for p in no_decay["params"])


def test_arena_adamw_cpu_matches_torch_adamw():
    m1, m2 = tiny_model(), tiny_model()
    arena = ParamArena(m1)
    opt1 = ArenaAdamW(arena, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    decay = [p for n, p in m2.named_parameters() if not ("norm" in n or "emb" in n or "bias" in n or p.dim() < 2)]
    rest = [p for n, p in m2.named_parameters() if ("norm" in n or "emb" in n or "bias" in n or p.dim() < 2)]
    opt2 = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}],
                             lr=1e-2, betas=(0.9, 0.95), eps=1e-8)
    x = torch.randint(0, 64, (2, 8))
    for _ in range(3):
        m1(x, labels=x)["loss"].backward()
        assert all(p.grad is None for p in m1.parameters())  # gradients live in the arena
        opt1.step()
        opt1.zero_grad()
        m2(x, labels=x)["loss"].backward()
        torch.nn.utils.clip_grad_norm_(m2.parameters(), 1.0)
        opt2.step()
        opt2.zero_grad()
    for (n, p), q in zip(m1.named_parameters(), m2.parameters()):
        assert torch.allclose(p, q, atol=2e-5), n
    sd = opt1.state_dict()
    opt1.load_state_dict(sd)
    assert sd["step"] == 3 and arena.num_params() == sum(p.numel() for p in m2.parameters())


def test_arena_lays_gate_and_up_projections_back_to_back():
    """The feed-forward registers w1, w2, w3 (the reference's order, which optimizer state follows); the arena still
    places w3 right behind w1, so that one ``[w1; w3]`` view serves the gate|up GEMM."""
    m = tiny_model()
    names = [n for n, _ in m.named_parameters()]
    i1, i2, i3 = (names.index(f"blocks.0.feed_forward.{w}.weight") for w in ("w1", "w2", "w3"))
    assert i1 < i2 < i3
    arena = ParamArena(m)
    for blk in m.blocks.values():
        ff = blk.feed_forward
        if not hasattr(ff, "w3") or not hasattr(ff.w1, "weight"):
            continue
        w13 = arena._fused_view([ff.w1.weight, ff.w3.weight])
        assert w13 is not None and torch.equal(w13, torch.cat([ff.w1.weight, ff.w3.weight], 0))
        assert w13.main_grad.shape == w13.shape and w13._covers[0] is ff.w1.weight
        att = blk.attention
        qkv = arena._fused_view([att.w_q.weight, att.w_k.weight, att.w_v.weight])
        assert qkv is not None and torch.equal(qkv, torch.cat([att.w_q.weight, att.w_k.weight, att.w_v.weight], 0))


def test_arena_view_fusion_pass_finds_every_gate_up_and_qkv_group():
    """The pass that the CUDA path runs at arena construction (``_fuse_views``; skipped on a CPU arena), run here on a
    bf16 CPU model by naming the device: every attention gets one ``[q; k; v]`` view and every feed-forward one
    ``[w1; w3]`` view, for the dense 1B shapes' ratios as for a hybrid MoE model (whose dense layers alternate with
    expert layers in the same regions)."""
    for moe in (False, True):
        torch.manual_seed(0)
        m = TransformerConfig(d_model=64, n_layers=4, n_heads=4, n_kv_heads=2, vocab_size=64, max_seq_len=16,
                              ffn_hidden=176, qk_norm=False, use_moe=moe, num_experts=4, moe_interval=2, moe_offset=1,
                              moe_hidden=64).build(dtype=torch.bfloat16)
        arena = ParamArena(m)
        arena.device = torch.device("cuda")      # only read by the pass; nothing here touches a GPU
        arena._fuse_views()
        n_ff = 0
        for blk in m.blocks.values():
            att = blk.attention
            assert att._fused_qkv is not None
            assert torch.equal(att._fused_qkv, torch.cat([att.w_q.weight, att.w_k.weight, att.w_v.weight], 0))
            ff = blk.feed_forward
            if hasattr(ff, "_fused_w13"):
                n_ff += 1
                assert ff._fused_w13 is not None, "gate and up projections are not adjacent in the arena"
                assert torch.equal(ff._fused_w13, torch.cat([ff.w1.weight, ff.w3.weight], 0))
        assert n_ff == (2 if moe else 4)


def test_diloco_compressor_roundtrip_and_error_feedback():
    ps = [torch.nn.Parameter(torch.zeros(1000))]
    before = torch.random.get_rng_state()
    c = DiLoCoCompressor(ps, compression_rank=16)
    assert torch.equal(before, torch.random.get_rng_state())  # the global RNG is left alone
    g = torch.randn(1000)
    comp, scale = c.compress(g)
    assert comp.shape == (16,)
    rec = c.decompress(comp, scale, 1000)
    assert rec.shape == (1000,) and torch.allclose(c.error_buffer, g - rec)   # the residual is carried over
    out = c.all_reduce_gradients(g)
    assert out.shape == (1000,)
    sd = c.compress_state_dict({"a": torch.randn(10, 50), "b": torch.randn(500)})
    assert sd["total_params"] == 1000 and sd["shapes"]["a"] == (10, 50)


# ------------------------------------------------------------------ checkpoints
def test_checkpoint_layout_roundtrip_and_retention(tmp_path):
    m = tiny_model()
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
    sched = CosineWithWarmup(opt, 2, 10)
    x = torch.randint(0, 64, (2, 8))
    m(x, labels=x)["loss"].backward()
    opt.step()
    sched.step()
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path), keep_last_n=2, incremental=False))
    ck.dataloader_tracker.update(4)
    for step in (10, 20, 30):
        d = ck.save(step, m, opt, scheduler=sched, extra={"tokens_seen": step * 16})
    assert sorted(os.listdir(tmp_path)) == ["step_000020", "step_000030"]
    files = sorted(os.listdir(d))
    assert files == ["metadata.json", "rank_0000_dataloader.json", "rank_0000_model.pt", "rank_0000_optimizer.pt",
                     "rank_0000_rng.pt", "rank_0000_scheduler.pt"]
    meta = json.load(open(os.path.join(d, "metadata.json")))
    assert meta["step"] == 30 and meta["version"] == 2 and meta["world_size"] == 1 and not meta["incremental"]
    assert "embeddings.weight" in meta["model_keys"] and meta["extra"]["tokens_seen"] == 480
    assert ck.latest_step() == 30
    m2 = tiny_model()
    with torch.no_grad():
        for p in m2.parameters():
            p.add_(1.0)
    opt2 = torch.optim.AdamW(m2.parameters(), lr=1e-2)
    sched2 = CosineWithWarmup(opt2, 2, 10)
    torch.manual_seed(123)
    got = ck.load(model=m2, optimizer=opt2, scheduler=sched2)
    assert got["step"] == 30 and sched2.last_epoch == sched.last_epoch
    for p, q in zip(m.parameters(), m2.parameters()):
        assert torch.equal(p, q)
    assert opt2.state_dict()["state"][0]["exp_avg"].abs().sum() > 0
    assert ck.dataloader_tracker.samples_seen == 4
    # overwrite vs suffix
    d2 = ck.save(30, m, opt)
    assert d2.name == "step_000030_1"      # a pathlib.Path, as the reference returns


def test_incremental_checkpoint_chain(tmp_path):
    m = tiny_model()
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path), incremental=True, keep_last_n=10,
                                                  full_save_interval=10, incremental_threshold=0.01))
    ck.save(1, m)
    with torch.no_grad():
        m.lm_head.weight.mul_(2.0)
        m.embeddings.weight.add_(1e-7)  # below the relative-change threshold
    d = ck.save(2, m)
    meta = json.load(open(os.path.join(d, "metadata.json")))
    delta = torch.load(os.path.join(d, "rank_0000_model.pt"), weights_only=False)
    assert meta["incremental"] and meta["base_checkpoint"] == "step_000001"
    assert "lm_head.weight" in delta and "embeddings.weight" not in delta and len(delta) < len(m.state_dict())
    m2 = tiny_model()
    ck.load(model=m2)
    assert torch.equal(m2.lm_head.weight, m.lm_head.weight)
    inc = IncrementalCheckpointer(0.01, 3)
    assert inc.should_save_full(0) and not inc.should_save_full(1) and inc.should_save_full(3)
    assert len(IncrementalCheckpointer._hash(torch.randn(100))) == 16


def test_retention_keeps_the_deltas_a_kept_checkpoint_needs(tmp_path):
    """keep_last_n = 2 with deltas: the delta of step 2 carries a change that steps 3 and 4 do not repeat, so it
    must survive the clean-up for step 4 to restore."""
    m = tiny_model()
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path), incremental=True, keep_last_n=2,
                                                  full_save_interval=10, incremental_threshold=0.01))
    ck.save(1, m)
    with torch.no_grad():
        m.lm_head.weight.mul_(2.0)
    ck.save(2, m)
    with torch.no_grad():
        m.embeddings.weight.mul_(3.0)
    ck.save(3, m)
    ck.save(4, m)
    assert os.path.isdir(tmp_path / "step_000001") and os.path.isdir(tmp_path / "step_000002")
    m2 = tiny_model()
    meta = ck.load(model=m2)
    assert meta["step"] == 4
    for k, v in m.state_dict().items():
        assert torch.equal(m2.state_dict()[k], v), k


def test_stager_gives_every_tensor_its_own_buffer():
    st = PinnedMemoryStager(enabled=False)
    sd = {f"l{i}.w": torch.full((4, 4), float(i)) for i in range(5)}
    out = st.stage_state_dict(sd)
    assert [float(out[f"l{i}.w"][0, 0]) for i in range(5)] == [0.0, 1.0, 2.0, 3.0, 4.0]
    st._buffer("a", torch.zeros(3))
    assert st._buffer("a", torch.zeros(3)) is st._buffer("a", torch.ones(3))          # reused across saves
    assert st._buffer("a", torch.zeros(3)) is not st._buffer("b", torch.zeros(3))    # never shared between names


def test_async_save_and_helpers(tmp_path):
    m = tiny_model()
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path), async_saves=True))
    fut = ck.save_async(5, m)
    ck.wait()
    assert fut.done() and os.path.isfile(tmp_path / "step_000005" / "metadata.json")
    ck.close()
    st = PinnedMemoryStager(enabled=True).stage_state_dict({"a": torch.ones(3), "n": {"b": torch.zeros(2)}, "k": 1})
    assert st["a"].device.type == "cpu" and st["n"]["b"].shape == (2,) and st["k"] == 1
    pc = PlanCache()
    sd = m.state_dict()
    assert pc.get(sd) is pc.get(sd) and pc.get(sd).total_bytes == sum(v.numel() * 4 for v in sd.values())


def _ckpt_worker(rank, world, save_dir):
    m = tiny_model()
    with torch.no_grad():
        m.lm_head.weight.fill_(float(rank))
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=save_dir))
    d = ck.save(7, m)
    files = sorted(os.listdir(d))
    assert "rank_0000_model.pt" in files and "rank_0001_model.pt" in files and "metadata.json" in files
    assert not any(f.startswith(".tmp") for f in os.listdir(save_dir))
    m2 = tiny_model()
    meta = ck.load(model=m2)
    assert meta["world_size"] == 2 and float(m2.lm_head.weight[0, 0]) == float(rank)
    return True


def test_checkpoint_two_ranks_single_directory(tmp_path):
    assert all(run_distributed(_ckpt_worker, 2, str(tmp_path)))


def test_fault_tolerant_checkpointer_skips_truncated_shard(tmp_path):
    m = tiny_model()
    opt = torch.optim.AdamW(m.parameters(), lr=1e-2)
    ft = FaultTolerantCheckpointer(str(tmp_path), save_interval=5, keep_last_n=5, async_save=False)
    assert ft.save(3, m, opt) is None and ft.should_save(5)
    ft.save(5, m, opt)
    with torch.no_grad():
        m.lm_head.weight.add_(1.0)
    ft.save(10, m, opt)
    meta = json.load(open(tmp_path / "step_000010" / "metadata.json"))
    assert set(meta) == {"step", "timestamp", "extra"}
    with open(tmp_path / "step_000010" / "rank_0000_model.pt", "r+b") as f:  # simulate a crash mid-write
        f.truncate(100)
    m2 = tiny_model()
    assert ft.resume(m2, torch.optim.AdamW(m2.parameters())) == 5
    os.makedirs(tmp_path / "step_000099")  # no metadata: ignored
    assert ft.find_latest_checkpoint() == 5 and ft.find_latest_checkpoint_dir().endswith("step_000005")
    assert FaultTolerantCheckpointer(str(tmp_path / "empty")).resume(m2) == 0


# ------------------------------------------------------------------ hang detection
def test_hang_detector_fires_and_heartbeat_prevents():
    fired = []
    hd = HangDetector(timeout=0.3, check_interval=0.05, on_hang=lambda: fired.append(1), abort_on_hang=False)
    hd.start()
    for _ in range(8):
        time.sleep(0.05)
        hd.heartbeat()
    assert not fired
    time.sleep(0.6)
    hd.stop()
    assert fired and hd.hang_detected
    def timed_out():
        raise RuntimeError("NCCL watchdog timeout")

    assert hd.check_collective_timeout(timed_out, timeout=1.0) is True and hd.check_collective_timeout(lambda: 3) is False
    with pytest.raises(CommTimeoutError):
        HangDetector.check_collective_timeout(timed_out, raise_on_timeout=True)
    with pytest.raises(ValueError):
        HangDetector.check_collective_timeout(lambda: (_ for _ in ()).throw(ValueError("other")))


def test_heartbeat_coordinator_detects_stalled_rank():
    from nanopysche_b200.fault_tolerance.hang_detection import _DictStore

    store = _DictStore()
    stalls = []
    ranks = [HeartbeatCoordinator(check_interval=0.05, hang_timeout=0.2, store=store, rank=r, world_size=3,
                                  on_stall=stalls.append) for r in range(3)]
    ranks[0].start()
    for step in range(1, 12):
        ranks[0].heartbeat(step)
        ranks[1].heartbeat(step)  # rank 2 never beats: its message is "dropped"
        time.sleep(0.05)
    ranks[0].stop()
    assert stalls and stalls[0] == [2]


def _hb_worker(rank, world):
    hb = HeartbeatCoordinator(check_interval=0.05, hang_timeout=0.3)
    assert hb.world_size == world
    for s in range(1, 6):
        if rank == 0 or s < 2:  # rank 1 stops making progress after its first step
            hb.heartbeat(s)
        time.sleep(0.1)
    stalled = []
    if rank == 0:
        hb.sync_heartbeats()
    time.sleep(0.35)
    if rank == 0:
        hb.heartbeat(99)
        counters = hb.sync_heartbeats()
        assert counters[0] == 99 and counters[1] == 1      # every rank's counter, as the reference returns them
        stalled = hb.stalled_ranks
    import torch.distributed as dist
    dist.barrier()
    return stalled


def test_heartbeat_over_process_group_store():
    res = run_distributed(_hb_worker, 2)
    assert res[0] == [1]


def test_profiler_callback_window(tmp_path):
    m = tiny_model()
    opt = torch.optim.SGD(m.parameters(), lr=0.01)
    prof = ProfilerCallback(save_dir=str(tmp_path), skip_first=1, wait=0, warmup=0, active=2)
    tc = TrainingConfig(global_batch_size=32, micro_batch_size=2, sequence_length=16, max_steps=5, log_interval=0,
                        save_interval=0, dtype=torch.float32, vocab_size=64)
    Trainer(tc, m, opt, None, None, [prof]).fit()
    assert any(f.endswith(".chrome_trace.json.gz") for f in os.listdir(tmp_path))


def _ft_resume_worker(rank, world, save_dir):
    """Rank 1's newest shard is truncated: both ranks must fall back to the older step together."""
    from nanopysche_b200.fault_tolerance.checkpoint import FaultTolerantCheckpointer

    m = tiny_model()
    ck = FaultTolerantCheckpointer(save_dir, save_interval=1, keep_last_n=5, async_save=False)
    ck.save(1, m, force=True)
    ck.save(2, m, force=True)
    dist.barrier()
    if rank == 1:
        with open(os.path.join(save_dir, "step_000002", "rank_0001_model.pt"), "wb") as f:
            f.write(b"trunc")
    dist.barrier()
    step = ck.resume(tiny_model())
    return step


def test_fault_tolerant_resume_agrees_across_ranks(tmp_path):
    assert run_distributed(_ft_resume_worker, 2, str(tmp_path)) == [1, 1]


def _compressed_dp_worker(rank, world):
    torch.manual_seed(0)
    m = tiny_model()
    m._replica_group = dist.group.WORLD
    opt = torch.optim.SGD(m.parameters(), lr=1e-2)
    tc = TrainingConfig(global_batch_size=2 * 16 * world, micro_batch_size=2, sequence_length=16, max_steps=3,
                        log_interval=0, save_interval=0, dtype=torch.float32, vocab_size=64, dp_world_size=world,
                        enable_gradient_compression=True, compression_rank=64)
    tr = Trainer(tc, m, opt, None, None, [])
    sent = []
    orig = dist.all_reduce

    def spy(t, *a, **k):
        sent.append(t.numel())
        return orig(t, *a, **k)

    dist.all_reduce = spy
    try:
        torch.manual_seed(100 + rank)       # every rank trains on its own batches
        tr.fit()
    finally:
        dist.all_reduce = orig
    assert 64 in sent and max(sent) <= 64, sent       # only the projection crosses the ranks
    assert tr._compressor.error_buffer.abs().sum() > 0
    flat = torch.cat([p.detach().reshape(-1) for p in m.parameters()])
    both = [torch.zeros_like(flat) for _ in range(world)]
    dist.all_gather(both, flat)
    assert torch.equal(both[0], both[1])               # identical updates: the replicas stay in step
    return True


def test_trainer_applies_gradient_compression_across_replicas():
    assert all(run_distributed(_compressed_dp_worker, 2))


def test_gradient_compression_refuses_sharded_optimizers():
    m = tiny_model()
    arena = ParamArena(m, device=torch.device("cpu"))
    opt = ArenaAdamW(arena, lr=1e-3)
    tc = TrainingConfig(global_batch_size=32, micro_batch_size=2, sequence_length=16, max_steps=1,
                        dtype=torch.float32, vocab_size=64, enable_gradient_compression=True)
    with pytest.raises(ValueError, match="un-sharded"):
        Trainer(tc, m, opt, None, None, [])


def test_speed_monitor_reads_device_time_one_step_late_and_normalises_per_device(monkeypatch):
    """With a (faked) CUDA device the step time comes from event pairs read one step later, and the per-device
    figures divide by the world size / replica count instead of charging the global batch to one device."""
    import nanopysche_b200.train.callbacks.speed_monitor as sm

    clock = {"t": 0.0}

    class FakeEvent:
        def __init__(self, enable_timing=False):
            self.t = None

        def record(self):
            self.t = clock["t"]

        def query(self):
            return False                      # never complete "yet": only older steps are read, after synchronize()

        def synchronize(self):
            pass

        def elapsed_time(self, other):
            return (other.t - self.t) * 1e3

    monkeypatch.setattr(sm.torch.cuda, "Event", FakeEvent)
    monkeypatch.setattr(sm.torch.cuda, "is_available", lambda: True)
    monkeypatch.setattr(sm, "_get_device_peak_flops", lambda d: 1e15)

    class T:
        device = torch.device("cuda", 0)
        world_size = 8
        tokens_per_step = 8 * 4096
        model = torch.nn.Linear(10, 10, bias=False)     # 100 parameters
        config = type("C", (), {"dp_world_size": 8, "cp_size": 1, "global_batch_size": 8 * 4096})()

        def __init__(self):
            self.m = {}

        def record_metric(self, k, v):
            self.m[k] = v

    t, cb = T(), SpeedMonitorCallback()
    for step in range(3):
        cb.pre_load_batch(t)
        cb.pre_step(t, None)
        clock["t"] += 0.5                    # the device takes 0.5 s per step; the host returns at once
        cb.post_step(t)
    # step 3 reports the device time of step 2
    assert abs(t.m["throughput/device/BPS"] - 2.0) < 1e-6
    assert abs(t.m["throughput/device/TPS"] - 4096 / 0.5) < 1e-3
    assert abs(t.m["throughput/device/flopsPS"] - 6 * 100 * 4096 / 0.5) < 1e-3
    assert t.m["throughput/total tokens"] == 3 * 8 * 4096


def test_arena_optimizer_state_reshards_to_another_world_size(tmp_path):
    """Elastic resume: the optimizer state of a 4-rank run with the bucketed shard layout (and of a 2-rank run with the
    contiguous one) is put together and cut again for this process's layout; the shard helpers are inverse to each
    other for every layout; an expert-sharded region refuses a changed world size."""
    from nanopysche_b200.optim.arena import assemble_shards, owned_slice

    flat = torch.arange(2 * 4 * 6, dtype=torch.float32)
    for world, bucket in ((4, 24), (2, 0), (4, 0), (2, 12), (1, 0)):
        parts = [owned_slice(flat, world, r, bucket) for r in range(world)]
        assert sum(p.numel() for p in parts) == flat.numel()
        assert torch.equal(assemble_shards(parts, bucket), flat)
    assert torch.equal(owned_slice(flat, 4, 1, 24), torch.cat([flat[6:12], flat[30:36]]))   # slice 1 of both buckets

    torch.manual_seed(0)
    m = tiny_model()
    arena = ParamArena(m, device=torch.device("cpu"))
    opt = ArenaAdamW(arena, lr=1e-3)
    want = {}
    for k, r in arena.regions.items():
        r.m.copy_(torch.randn_like(r.m))
        r.v.copy_(torch.rand_like(r.v))
        want[k] = (r.m.clone(), r.v.clone())
    full_sd = opt.state_dict()
    full_sd["step"] = 7

    def fake_run(world, bucket_of):
        """What the ranks of a ``world``-way sharded run would have saved for this optimizer state."""
        out = []
        for rank in range(world):
            regs = {}
            for k, r in arena.regions.items():
                b = bucket_of(r)
                total = (r.numel + max(b, 4 * world) - 1) // max(b, 4 * world) * max(b, 4 * world)
                ent = {"master": None, "lo": 0, "cnt": total // world, "bucket": b}
                for name in ("m", "v"):
                    pad = torch.zeros(total)
                    pad[:r.numel] = getattr(r, name)[:r.numel]
                    ent[name] = owned_slice(pad, world, rank, b).clone()
                regs[k] = ent
            lay = {"world": world, "rank": rank,
                   "regions": {k: {"numel": r.numel, "total": 0, "replicated": True, "sharded": True}
                               for k, r in arena.regions.items()}}
            out.append({"step": 7, "param_groups": full_sd["param_groups"], "regions": regs, "layout": lay})
        return out

    for world, bucket_of in ((4, lambda r: 64), (2, lambda r: 0)):
        saved = fake_run(world, bucket_of)
        for r in arena.regions.values():
            r.m.zero_()
            r.v.zero_()
        opt.load_state_dict_resharded(saved)
        assert opt.step_count == 7
        for k, r in arena.regions.items():
            assert torch.equal(r.m[:r.numel], want[k][0][:r.numel]) and torch.equal(r.v[:r.numel], want[k][1][:r.numel])

    # through the checkpointer: a directory written by a 2-rank run, read by this single process
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path), pinned_memory=False))
    ck.save(7, m, opt)
    step_dir = ck._find_latest_checkpoint()
    meta_path = os.path.join(step_dir, "metadata.json")
    meta = json.load(open(meta_path))
    meta["world_size"] = 2
    json.dump(meta, open(meta_path, "w"))
    for rank, sd in enumerate(fake_run(2, lambda r: 0)):
        torch.save(sd, os.path.join(step_dir, f"rank_{rank:04d}_optimizer.pt"))
    bad = fake_run(2, lambda r: 0)
    for r in arena.regions.values():
        r.m.zero_()
    ck.load(step_dir, m, opt)
    for k, r in arena.regions.items():
        assert torch.equal(r.m[:r.numel], want[k][0][:r.numel])

    # expert-sharded regions cannot follow a changed world size
    key = next(iter(arena.regions))
    arena.regions[key].replicated = False
    arena.world = 1
    with pytest.raises(ValueError, match="expert-sharded"):
        opt.load_state_dict_resharded(bad)


def _departure_worker(rank, world, save_dir):
    """Rank 2 announces in ``pre_step`` of its third step that this is its last one and returns from ``fit()`` after
    it; ranks 0 and 1 find the note at the top of step four - before any collective that would wait for rank 2 -
    raise ``PeerLeftError``, run ``on_error`` and write their emergency checkpoints. Nothing hangs: every collective
    that was started had all three ranks in it."""
    from nanopysche_b200.fault_tolerance import HeartbeatCoordinator, PeerLeftError

    torch.manual_seed(0)
    m = tiny_model()
    m._replica_group = dist.group.WORLD
    m._needs_grad_sync = True
    opt = torch.optim.SGD(m.parameters(), lr=1e-2)
    events = []

    class Leaver(Callback):
        def pre_step(self, trainer, batch):
            if trainer.rank == 2 and trainer.step == 2:
                trainer.leave_after_step()            # the step about to run (number 3) is the last one

        def on_error(self, trainer, err):
            events.append(type(err).__name__)

    tc = TrainingConfig(global_batch_size=2 * 16 * world, micro_batch_size=2, sequence_length=16, max_steps=8,
                        log_interval=0, save_interval=0, dtype=torch.float32, vocab_size=64, dp_world_size=world,
                        save_dir=save_dir)
    tr = Trainer(tc, m, opt, None, None, [Leaver()], heartbeat=HeartbeatCoordinator(check_interval=60.0))
    err = None
    try:
        tr.fit()
    except PeerLeftError as e:
        err = str(e)
    return rank, tr.step, err, events, tr.emergency_checkpoint_dir


def test_planned_departure_stops_the_peers_before_the_next_step(tmp_path):
    res = sorted(run_distributed(_departure_worker, 3, str(tmp_path)))
    (r0, s0, e0, ev0, d0), (r1, s1, e1, ev1, d1), (r2, s2, e2, ev2, d2) = res
    assert (s0, s1, s2) == (3, 3, 3)                      # everyone completed exactly three steps
    assert e2 is None and ev2 == [] and d2 == d0           # the leaver returned normally, its state saved with the others
    for e, ev, d in ((e0, ev0, d0), (e1, ev1, d1)):
        assert e is not None and "[2]" in e and ev == ["PeerLeftError"]
        assert d is not None and os.path.isdir(d)
    assert os.path.exists(os.path.join(d0, "rank_0000_model.pt")) and os.path.exists(os.path.join(d1, "rank_0001_model.pt"))
    assert os.path.exists(os.path.join(d0, "rank_0002_optimizer.pt"))
    # the directory loads like a regular checkpoint, here into a single process (another world size)
    meta = json.load(open(os.path.join(d0, "metadata.json")))
    assert meta["step"] == 3 and meta["world_size"] == 3
    m = tiny_model()
    opt = torch.optim.SGD(m.parameters(), lr=1e-2)
    DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path))).load(d0, m, opt, restore_rng=False)
    saved = torch.load(os.path.join(d0, "rank_0000_model.pt"))
    for k, v in m.state_dict().items():
        assert torch.equal(v, saved[k]), k


def test_reference_method_surface_of_checkpoint_and_pipeline_helpers(tmp_path):
    """Methods a user of the reference may call on the helper classes (names and meaning as in
    checkpoint/distributed.py and distributed/pipeline_runtime.py of the reference)."""
    from nanopysche_b200.checkpoint.distributed import (DataloaderStateTracker, IncrementalCheckpointer, PlanCache,
                                                        SavePlan)
    from nanopysche_b200.fp8.training import FP8Config
    from nanopysche_b200.parallel.pipeline_runtime import PipelineParallelConfig, PipelineSplitStyle

    st = PinnedMemoryStager()
    t = torch.arange(6.0).view(2, 3)
    out = st.stage_tensor(t)
    assert torch.equal(out, t) and out.data_ptr() != t.data_ptr()

    pc = PlanCache()
    assert pc.get_plan(1) is None
    plan = pc.get({"a": torch.zeros(3)})
    assert pc.get_plan(5) is plan
    pc.cache_plan(7, SavePlan(["x"], {"x": 4}, 4))
    assert pc.get_plan(7).keys == ["x"]
    pc.invalidate()
    assert pc.get_plan(7) is None

    inc = IncrementalCheckpointer(full_save_interval=4)
    assert inc.compute_param_hash(t) == inc.compute_param_hash(t.clone()) != inc.compute_param_hash(t + 1)
    assert inc.is_base_checkpoint_needed(8) and not inc.is_base_checkpoint_needed(9) and inc.is_base_checkpoint_needed(9, 3)

    tr = DataloaderStateTracker()
    tr.update(4)
    tr.update(current_file="shard_3.bin", global_step=11)          # the reference's keyword form: fields, no count
    assert tr.get_state()["samples_seen"] == 4 and tr.get_state()["extra"]["current_file"] == "shard_3.bin"
    p = os.path.join(str(tmp_path), "dl.json")
    tr.save(p)
    tr2 = DataloaderStateTracker()
    tr2.load(p)
    assert tr2.state_dict() == tr.state_dict()

    cfg = PipelineParallelConfig(4, schedule="ZBVZeroBubble")
    assert cfg.stages_per_rank == 2 and cfg.stages_per_rank() == 2 and cfg.total_stages == 8
    assert not cfg.is_single_stage and cfg.split_style == PipelineSplitStyle.v
    assert PipelineParallelConfig(2).is_single_stage and PipelineParallelConfig(2).total_stages == 2
    assert FP8Config(enabled=True).build_torchao_config() is None

    m = tiny_model()
    tc = TrainingConfig(global_batch_size=32, micro_batch_size=2, sequence_length=16, max_steps=1, dtype=torch.float32,
                        vocab_size=64)
    assert Trainer(tc, m, torch.optim.SGD(m.parameters(), lr=0.1), None, None, []).get_vocab_size() == 64


def _loader_coords_worker(rank, world):
    """The loader is built before the mesh (as the CLI does) and resolves its data-parallel index at the first batch:
    with dp 2 x tp 2 the tensor-parallel peers read the same rows, the data-parallel peers different ones."""
    from nanopysche_b200.parallel.mesh import build_world_mesh

    tokens = np.arange(64 * 17, dtype=np.int64)
    loader = create_distributed_loader(tokens, 2, 16, shuffle=False)
    mesh = build_world_mesh(tp_size=2, device_type="cpu", replace=True)
    ids, _ = next(iter(loader))
    assert (loader.dp_rank, loader.dp_world) == (mesh["dp"].get_local_rank(), 2)
    first = [torch.zeros_like(ids[0]) for _ in range(world)]
    dist.all_gather(first, ids[0].contiguous())
    tp_peer, dp_peer = rank ^ 1, rank ^ 2
    assert torch.equal(first[rank], first[tp_peer]) and not torch.equal(first[rank], first[dp_peer])
    return True


def test_loader_built_before_the_mesh_follows_the_mesh():
    assert all(run_distributed(_loader_coords_worker, 4))
