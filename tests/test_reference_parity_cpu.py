"""Numerical parity with the unmodified reference on CPU, in fp32: the reference (installed under ``baseline/_ref``)
runs in a child process (``tests/reference_oracle.py``) and writes weights, inputs and results; here the same weights
go into this package's classes through ``load_state_dict`` - the state-dict keys and layouts are the reference's, which
is what lets a checkpoint move between the two - and logits, loss and every gradient are compared. Also the LR
schedules, RoPE tables, AdamW update and the decay / no-decay parameter split. Skipped when the reference is not
installed."""
import os
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import reference_oracle as oracle  # noqa: E402  (only its case tables and builder; it imports nothing of either package)


@pytest.fixture(scope="module")
def ref(tmp_path_factory):
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "nanopsyche")):
        pytest.skip("the reference is not installed under baseline/_ref")
    out = str(tmp_path_factory.mktemp("oracle") / "ref.pt")
    env = dict(os.environ, PYTHONPATH="")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "reference_oracle.py"), out], env=env,
                       capture_output=True, text=True, timeout=600)
    if r.returncode == 3:
        pytest.skip("the reference is not installed under baseline/_ref")
    assert r.returncode == 0, r.stderr[-2000:]
    return torch.load(out, weights_only=False)


@pytest.mark.parametrize("case", list(oracle.MODEL_CASES))
def test_model_matches_the_reference(ref, case):
    from nanopysche_b200.models import moe as our_moe
    from nanopysche_b200.models.transformer import Transformer

    want = ref["models"][case]
    model = oracle.build(Transformer, our_moe, case, seed=99)      # other initial weights: everything comes from the load
    # same keys in the same order: torch optimizers store their state by parameter position
    assert list(model.state_dict().keys()) == list(want["state_dict"].keys())
    for k, v in model.state_dict().items():
        assert v.shape == want["state_dict"][k].shape, k
    model.load_state_dict(want["state_dict"], strict=True)
    for k, v in model.state_dict().items():                          # and what is written back is what was read
        assert torch.equal(v, want["state_dict"][k]), k
    got = oracle.run_model(model, ref["ids"])
    assert torch.allclose(got["logits"], want["logits"], atol=2e-5, rtol=1e-4), case
    assert abs(float(got["loss"]) - float(want["loss"])) < 1e-5
    if case.startswith("dense"):
        assert got["keys"] == want["keys"] == ["logits", "loss"]       # no "aux_loss" entry without MoE layers
    grads = {n: p.grad for n, p in model.named_parameters()}
    assert list(grads) == [k for k in want["state_dict"] if k in grads]
    assert set(want["grads"]) <= set(grads)
    for n, g in want["grads"].items():
        assert grads[n] is not None, n
        scale = g.abs().max().item() + 1e-12
        assert (grads[n] - g).abs().max().item() / scale < 2e-4, (case, n)


def test_lr_schedules_match_the_reference(ref):
    from nanopysche_b200.train import scheduler as S

    s = ref["sched"]
    for name, fn in (("cosine", lambda t: S.cosine_with_warmup(t, 10, 100, 1e-5, 3e-4)),
                     ("wsd", lambda t: S.warmup_stable_decay(t, 10, 50, 40, 1e-5, 3e-4)),
                     ("exp", lambda t: S.exponential_decay(t, 10, 0.97, 1e-5, 3e-4))):
        for t, want in zip(s["steps"], s[name]):
            assert fn(t) == pytest.approx(want, rel=1e-12, abs=1e-15), (name, t)
    for name, make in (("CosineWithWarmup", lambda o: S.CosineWithWarmup(o, warmup_steps=5, max_steps=40)),
                       ("WarmupStableDecay", lambda o: S.WarmupStableDecay(o, warmup_steps=5, stable_steps=20,
                                                                           decay_steps=15))):
        p = torch.nn.Parameter(torch.zeros(2))
        opt = torch.optim.SGD([p], lr=3e-4)
        sch = make(opt)
        for want in s[name]:
            assert opt.param_groups[0]["lr"] == pytest.approx(want, rel=1e-12, abs=1e-18), name
            opt.step()
            sch.step()


def test_rope_tables_and_rotation_match_the_reference(ref):
    from nanopysche_b200.models import rope as R

    kws = {"plain": dict(base=10000.0), "theta_500k": dict(base=500000.0),
           "partial": dict(base=10000.0, partial_rotary_factor=0.5),
           "scaled": dict(base=500000.0, scaling=R.RoPEScalingConfig(factor=8.0, low_freq_factor=1.0,
                                                                     high_freq_factor=4.0,
                                                                     original_max_position_embeddings=64))}
    for name, kw in kws.items():
        want = ref["rope"][name]
        rope = R.RotaryEmbedding(32, max_seq_len=256, **kw)
        cos, sin = rope(48, offset=7, device=torch.device("cpu"))
        assert cos.shape == want["cos"].shape, name
        assert torch.allclose(cos, want["cos"], atol=2e-6) and torch.allclose(sin, want["sin"], atol=2e-6), name
        if want["y"] is not None:
            y = R.apply_rotary_emb(want["x"], cos, sin)
            assert torch.allclose(y, want["y"], atol=1e-5), name


def test_adamw_and_parameter_groups_match_the_reference(ref):
    from nanopysche_b200.models import moe as our_moe
    from nanopysche_b200.models.transformer import Transformer
    from nanopysche_b200.optim.adamw import AdamW, create_adamw

    a = ref["adamw"]
    m = oracle.build(Transformer, our_moe, "moe_gate_bias")
    opt = create_adamw(m, lr=1e-2, weight_decay=0.1)
    groups = [sorted(n for n, p in m.named_parameters() if any(p is q for q in grp["params"]))
              for grp in opt.param_groups]
    assert [g["weight_decay"] for g in opt.param_groups] == [0.1, 0.0]
    assert groups == a["groups"]
    ws = [torch.nn.Parameter(w.clone()) for w in a["w0"]]
    opt = AdamW([{"params": [ws[0]], "weight_decay": 0.1}, {"params": [ws[1]], "weight_decay": 0.0}], lr=1e-2,
                betas=(0.9, 0.95), eps=1e-8)
    for gs in a["grads"]:
        for w, g in zip(ws, gs):
            w.grad = g.clone()
        opt.step()
    for w, want in zip(ws, a["w"]):
        assert torch.allclose(w, want, atol=1e-6, rtol=1e-5)


def test_trainer_trajectory_matches_the_reference(ref):
    """Six optimizer steps through ``Trainer._train_step_with_callbacks`` - gradient accumulation over two micro-batches,
    clipping, AdamW with the decay split, warm-up and cosine schedule, batches in the reference's mapping format - end in
    the same weights. The logged loss is the mean over the micro-batches here; the reference logs their sum
    (train/trainer.py:326-333 multiplies the already divided loss back by the accumulation count)."""
    from nanopysche_b200.models import moe as our_moe
    from nanopysche_b200.models.transformer import Transformer
    from nanopysche_b200.optim.adamw import create_adamw
    from nanopysche_b200.train.scheduler import CosineWithWarmup
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig

    t = ref["trainer"]
    m = oracle.build(Transformer, our_moe, "dense", seed=77)
    m.load_state_dict(t["init"])
    losses, final = oracle.run_trainer(m, t["batches"], Trainer, TrainingConfig, CosineWithWarmup, create_adamw)
    for a, b in zip(losses, t["losses"]):
        assert a == pytest.approx(b / oracle.ACCUM, rel=1e-5)
    for k, v in t["final"].items():
        assert torch.allclose(final[k], v, atol=1e-5, rtol=1e-4), k


def test_checkpoint_written_by_the_reference_loads_here(ref, tmp_path):
    """A checkpoint directory from the reference's ``DistributedCheckpointer`` (model with MoE layers and shared
    experts, its AdamW, its scheduler) restores model, optimizer moments and schedule position here; saving again in the
    reference's positional order ``save(model, optimizer, scheduler, step)`` writes the same file set."""
    from nanopysche_b200.checkpoint.distributed import CheckpointConfig, DistributedCheckpointer
    from nanopysche_b200.models import moe as our_moe
    from nanopysche_b200.models.transformer import Transformer
    from nanopysche_b200.optim.adamw import create_adamw
    from nanopysche_b200.train.scheduler import CosineWithWarmup

    c = ref["checkpoint"]
    m = oracle.build(Transformer, our_moe, "moe_shared_expert", seed=123)
    opt = create_adamw(m, lr=1e-2, weight_decay=0.1)
    sch = CosineWithWarmup(opt, warmup_steps=2, max_steps=6)
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=c["dir"], pinned_memory=False))
    meta = ck.load(model=m, optimizer=opt, scheduler=sch)
    assert meta["step"] == 3 and meta["extra"]["tokens_seen"] == 192
    for k, v in m.state_dict().items():
        assert torch.equal(v, c["model"][k]), k
    assert sch.last_epoch == c["last_epoch"] and opt.param_groups[0]["lr"] == pytest.approx(c["lr"])
    for p_, st in opt.state.items():                     # every moment landed on the parameter of its shape
        assert st["exp_avg"].shape == p_.shape
    m.train()
    m(ref["ids"], labels=ref["ids"])["loss"].backward()  # the resumed run's next step equals the reference's
    opt.step()
    for k, v in m.state_dict().items():
        assert torch.allclose(v, c["after_next_step"][k], atol=1e-6, rtol=1e-5), k
    ck2 = DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path), pinned_memory=False))
    opt.zero_grad()
    d = ck2.save(m, opt, sch, 4, None, {"tokens_seen": 256})
    assert os.path.basename(d) == "step_000004"
    want_files = {f for f in os.listdir(os.path.join(c["dir"], "step_000003")) if not f.endswith("dataloader.json")}
    assert want_files <= set(os.listdir(d))


def test_fit_emits_the_reference_metric_names_and_hook_order(ref, tmp_path):
    """``Trainer.fit()`` on its own synthetic batches with the stock monitor callbacks: every metric name the
    reference's run reports is reported here, and the lifecycle hooks fire in the reference's order (plus ``pre_step``
    and ``post_train``, which the reference declares in its base class and never calls)."""
    from nanopysche_b200.models import moe as our_moe
    from nanopysche_b200.models.transformer import Transformer
    from nanopysche_b200.optim.adamw import create_adamw
    from nanopysche_b200.train.callbacks import (GPUMemoryMonitorCallback, SpeedMonitorCallback,
                                                 StabilityMonitorCallback)
    from nanopysche_b200.train.callbacks.base import Callback
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig

    names, events = oracle.run_fit_with_callbacks(
        oracle.build(Transformer, our_moe, "dense"), Trainer, TrainingConfig, Callback,
        [SpeedMonitorCallback, StabilityMonitorCallback, GPUMemoryMonitorCallback], create_adamw, str(tmp_path))
    assert set(ref["fit"]["metric_names"]) <= set(names), set(ref["fit"]["metric_names"]) - set(names)
    assert [e for e in events if e not in ("pre_step", "post_train")] == ref["fit"]["events"]
    assert events.count("pre_step") == 3 and events[-2:] == ["post_train", "close"]


def test_moe_layer_over_several_steps_matches_the_reference(ref):
    """Eight training forwards of a MoE layer with capacity drops and adaptive capacity: outputs, per-expert drop
    counts, the adapted capacity factor and its drop-rate average follow the reference step by step. With the score bias
    on, the reference's update ``bias += gamma * (count / tokens - 1 / E)`` is, up to a shift common to all experts
    (which top-k selection and softmax gating do not see), this package's ``sign * gamma * (count / assignments - 1 / E)``
    with ``sign = +1`` and ``gamma`` times top-k: run that way, routing and outputs stay the reference's."""
    from nanopysche_b200.models import moe as our_moe

    q = ref["moe_sequence"]
    _, rows = oracle.run_moe_sequence(our_moe, q["state_dict"])
    for i, (a, b) in enumerate(zip(rows, q["rows"])):
        assert torch.allclose(a["y"], b["y"], atol=1e-6), i
        assert a["per_expert"] == b["per_expert"] and a["routed"] == b["routed"], i
        assert a["capacity_factor"] == pytest.approx(b["capacity_factor"]) and a["ema"] == pytest.approx(b["ema"]), i
        assert a["aux"] == pytest.approx(b["aux"], rel=1e-5), i
    _, rows = oracle.run_moe_sequence(our_moe, q["state_dict_bias"], bias_gamma=0.05 * 2, sign=+1.0)
    for i, (a, b) in enumerate(zip(rows, q["rows_bias"])):
        assert torch.allclose(a["bias"] - a["bias"].mean(), b["bias"] - b["bias"].mean(), atol=1e-6), i
        assert torch.allclose(a["y"], b["y"], atol=1e-6), i
        assert a["per_expert"] == b["per_expert"], i


def test_fault_tolerant_checkpoint_of_the_reference_resumes_here(ref):
    from nanopysche_b200.fault_tolerance.checkpoint import FaultTolerantCheckpointer
    from nanopysche_b200.models import moe as our_moe
    from nanopysche_b200.models.transformer import Transformer
    from nanopysche_b200.optim.adamw import create_adamw

    f = ref["ft"]
    m = oracle.build(Transformer, our_moe, "moe_shared_expert", seed=31)
    opt = create_adamw(m, lr=1e-2, weight_decay=0.1)
    ft = FaultTolerantCheckpointer(f["dir"], save_interval=2, async_save=False)
    assert ft.find_latest_checkpoint() == f["latest"] == 4
    assert ft.resume(m, opt) == 4
    for k, v in m.state_dict().items():
        assert torch.equal(v, f["model"][k]), k
    for p_, st in opt.state.items():
        assert st["exp_avg"].shape == p_.shape


def test_attention_module_options_match_the_reference(ref):
    """Projection biases, qk-norm, full multi-head, scaled RoPE; causal, bidirectional and boolean-mask calls."""
    from nanopysche_b200.models.attention import Attention
    from nanopysche_b200.models.rope import RoPEScalingConfig

    got, _ = oracle.run_attention(Attention, RoPEScalingConfig, ref["attention"]["state_dicts"])
    for name, outs in ref["attention"]["out"].items():
        for call, want in outs.items():
            assert torch.allclose(got[name][call], want, atol=1e-6), (name, call)


def _tp_worker(rank, world, full_path, out_dir):
    from torch.distributed.device_mesh import init_device_mesh

    from nanopysche_b200.models.transformer import Transformer

    mesh = init_device_mesh("cpu", (world,), mesh_dim_names=("tp",))
    r = oracle.tp_rank_result(Transformer, torch.load(full_path), mesh["tp"])
    del r["full"]
    torch.save(r, os.path.join(out_dir, f"ours_tp_rank{rank}.pt"))     # tensors go through a file, not the result queue
    return True


def test_tensor_parallel_shards_are_the_reference_s(ref, tmp_path):
    """Two gloo ranks, Megatron TP of a GQA model (8 query / 4 KV heads): from the same full weights both code bases cut
    the same shards under the same keys - a checkpoint of a tensor-parallel run moves over rank by rank - and compute
    the same loss. The gradients here equal the single-process model's; the reference's do not (its column-parallel
    projections have no all-reduce of the input gradient in the backward pass - it uses only the output-side operator,
    model/attention.py:191-192, model/feed_forward.py:77-78 - so everything upstream of a sharded layer sees a
    partial gradient), which this test pins so that the difference stays a known one."""
    from conftest import run_distributed

    from nanopysche_b200.models.transformer import Transformer

    want = ref["tp"]
    full_sd = want[0]["full"]
    torch.save(full_sd, tmp_path / "full.pt")
    assert all(run_distributed(_tp_worker, 2, str(tmp_path / "full.pt"), str(tmp_path)))
    got = [torch.load(tmp_path / f"ours_tp_rank{r}.pt") for r in range(2)]
    torch.manual_seed(0)
    single = Transformer(**oracle.BASE, block=dict(oracle.TP_BLOCK))
    single.load_state_dict(full_sd)
    ids = torch.arange(2 * 16).reshape(2, 16) % oracle.BASE["vocab_size"]
    single(ids, labels=ids)["loss"].backward()
    full_grads = {n: p.grad for n, p in single.named_parameters()}
    for rank in range(2):
        a, b = got[rank], want[rank]
        assert list(a["shards"]) == list(b["shards"])
        for k, v in a["shards"].items():
            assert v.shape == b["shards"][k].shape and torch.equal(v, b["shards"][k]), (rank, k)
        assert torch.allclose(a["loss"], b["loss"], atol=1e-5)
        for k in ("embeddings.weight", "blocks.0.attention_norm.weight", "blocks.1.feed_forward_norm.weight",
                  "lm_head.weight"):
            assert torch.allclose(a["grads"][k], full_grads[k], atol=1e-6), (rank, k)
        k = "blocks.0.feed_forward.w1.weight"          # column-parallel: this rank's rows of the full gradient
        rows = a["grads"][k].shape[0]
        assert torch.allclose(a["grads"][k], full_grads[k][rank * rows:(rank + 1) * rows], atol=1e-6)
        # the known difference: the reference's upstream gradients are partial sums
        assert not torch.allclose(b["grads"]["embeddings.weight"], full_grads["embeddings.weight"], atol=1e-4)


def test_routing_replay_matches_the_reference(ref):
    """R3 routing replay (``set_replay_mask`` / ``clear_replay_mask``): the replayed choice, the renormalised weights,
    the layer output and the gradients of router and input are the reference's; without the mask the router goes back
    to its own choice."""
    from nanopysche_b200.models import moe as our_moe

    want = ref["routing_replay"]["out"]
    _, got = oracle.run_routing_replay(our_moe, ref["routing_replay"]["state_dict"])
    assert torch.equal(got["idx"], want["idx"])
    assert torch.equal(got["idx_replayed"].sort(-1).values, want["idx_replayed"].sort(-1).values)
    assert torch.allclose(got["weights"].sort(-1).values, want["weights"].sort(-1).values, atol=1e-6)
    assert torch.allclose(got["y"], want["y"], atol=1e-6)
    assert torch.allclose(got["gate_grad"], want["gate_grad"], atol=1e-6)
    assert torch.allclose(got["x_grad"], want["x_grad"], atol=1e-6)
    assert torch.equal(got["idx_after_clear"].sort(-1).values, want["idx_after_clear"].sort(-1).values)


def test_moe_options_and_phase_api_match_the_reference(ref):
    """Seeded router jitter, L2-normalised expert weights, and the five-phase API of the hybrid block
    (route, dispatch, local_compute, combine, reassemble) with capacity drops and a shared expert: same kept tokens,
    same output as the layer's own forward, same as the reference."""
    from nanopysche_b200.models import moe as our_moe

    want = ref["moe_options"]["out"]
    got, _ = oracle.run_moe_options(our_moe, ref["moe_options"]["state_dicts"])
    assert torch.allclose(got["jitter"], want["jitter"], atol=1e-6)
    assert torch.allclose(got["l2"], want["l2"], atol=1e-6)
    a, b = got["phases"], want["phases"]
    assert a["kept"] == b["kept"] and torch.equal(a["keep"], b["keep"])
    assert torch.allclose(a["y"], b["y"], atol=1e-6) and torch.allclose(a["whole"], b["whole"], atol=1e-6)
    assert torch.allclose(a["y"], a["whole"], atol=1e-6) and a["aux"] == pytest.approx(b["aux"], rel=1e-5)


def test_feed_forward_and_rmsnorm_match_the_reference(ref):
    from nanopysche_b200.models.feed_forward import FeedForward
    from nanopysche_b200.models.norm import RMSNorm

    want = ref["small_modules"]["out"]
    got, _ = oracle.run_small_modules(FeedForward, RMSNorm, ref["small_modules"]["state_dicts"])
    for name, w in want.items():
        assert got[name].shape == w.shape, name
        if name == "norm_bf16":
            # "same dtype as input" says the reference's docstring; its code rebinds x to the fp32 copy before casting
            # back, so a bf16 input comes out fp32 (model/norm.py:38-50). Here the output has the input's dtype.
            assert got[name].dtype == torch.bfloat16 and w.dtype == torch.float32
        else:
            assert got[name].dtype == w.dtype, name
        tol = 1e-6 if got[name].dtype == torch.float32 else 2e-2
        assert torch.allclose(got[name].float(), w.float(), atol=tol, rtol=tol), name
