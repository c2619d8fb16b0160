"""End-to-end GPU checks: the fused MoE layer against the generic PyTorch path, the arena optimizer
against torch AdamW, and a short training run of the flagship architecture (GPU only)."""
import copy

import pytest
import torch

pytestmark = pytest.mark.gpu


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    from nanopysche_b200.ops import _lib

    yield
    torch.cuda.synchronize()
    _lib.check_status("after test")


@pytest.mark.parametrize("capacity,shared", [(1.25, False), (None, False), (1.25, True)])
def test_fused_moe_matches_generic_path(capacity, shared):
    from nanopysche_b200.models.moe import MoEBase
    from nanopysche_b200.ops.moe import build_runtime

    torch.manual_seed(0)
    B, S, D, H, E, K = 2, 256, 256, 256, 4, 2
    fused = MoEBase(d_model=D, hidden_size=H, num_experts=E, top_k=K, capacity_factor=capacity, dtype=torch.bfloat16,
                    device="cuda", init_std=0.05, shared_expert=shared)
    fused.router.cuda()
    ref = copy.deepcopy(fused).float()
    build_runtime([fused], tokens=B * S, device=torch.device("cuda"))
    assert fused._can_fuse(torch.empty(1, 1, D, device="cuda", dtype=torch.bfloat16))
    x = (torch.randn(B, S, D, device="cuda")).bfloat16()
    xa = x.clone().requires_grad_(True)
    y = fused(xa)
    gy = torch.randn_like(y)
    (y * gy).sum().backward()
    xb = x.float().requires_grad_(True)
    yr = ref(xb)
    (yr * gy.float()).sum().backward()
    assert fused.last_dropped == ref.last_dropped and fused.total_tokens_routed == B * S
    if capacity is not None:
        assert fused.last_dropped > 0 and fused.per_expert_drops.tolist() == ref.per_expert_drops.tolist()
    assert rel(y, yr) < 2e-2
    assert rel(xa.grad, xb.grad) < 3e-2
    for n in ("w1", "w2", "w3"):
        assert rel(getattr(fused, n).grad, getattr(ref, n).grad) < 3e-2, n
    assert rel(fused.router.gate.weight.grad, ref.router.gate.weight.grad) < 5e-2
    if shared:
        for n in ("w1", "w2", "w3"):
            assert rel(getattr(fused.shared_expert, n).grad, getattr(ref.shared_expert, n).grad) < 3e-2, n


def test_flagship_block_matches_fp32_reference_and_trains():
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.engine import prepare_training

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=2048, d_model=256, n_layers=2, n_heads=4, n_kv_heads=2, ffn_hidden=512,
                            rope_base=10000.0, max_seq_len=256, qk_norm=False, use_moe=True, num_experts=4,
                            moe_top_k=2, moe_interval=2, moe_offset=1, moe_hidden=256, moe_capacity_factor=None)
    model = cfg.build(dtype=torch.bfloat16, init_device="cuda")
    ref = copy.deepcopy(model).float()
    ids = torch.randint(0, 2048, (2, 256), device="cuda")
    opt, arena = prepare_training(model, tokens_per_rank=512, lr=2e-3)
    assert model.blocks["0"].attention._fused_qkv is not None and model.blocks["0"].feed_forward._fused_w13 is not None
    out = model(ids, labels=ids)
    outr = ref(ids, labels=ids)
    assert abs(out["loss"].item() - outr["loss"].item()) < 2e-2 * outr["loss"].item()
    (out["loss"] + out["aux_loss"]).backward()
    (outr["loss"] + outr["aux_loss"]).backward()
    g = dict(arena.named_main_grads())
    for name in ("blocks.0.attention.w_q.weight", "blocks.0.feed_forward.w2.weight", "blocks.1.moe.w1",
                 "blocks.0.attention_norm.weight", "embeddings.weight", "lm_head.weight"):
        assert rel(g[name], dict(ref.named_parameters())[name].grad) < 6e-2, name
    losses = []
    opt.step()
    opt.zero_grad()
    for _ in range(8):
        o = model(ids, labels=ids)
        (o["loss"] + o["aux_loss"]).backward()
        opt.step()
        opt.zero_grad()
        losses.append(o["loss"].item())
    assert losses[-1] < losses[0] - 0.5 and opt.last_grad_norm.item() > 0


def test_arena_adamw_gpu_matches_torch():
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.optim.arena import ArenaAdamW, ParamArena

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=512, d_model=128, n_layers=1, n_heads=2, ffn_hidden=256, max_seq_len=64,
                            qk_norm=False)
    m1 = cfg.build(dtype=torch.float32, init_device="cuda")
    m2 = copy.deepcopy(m1)
    arena = ParamArena(m1)
    o1 = ArenaAdamW(arena, lr=1e-2, weight_decay=0.1, max_grad_norm=1.0)
    decay = [p for n, p in m2.named_parameters() if not ("norm" in n or "emb" in n or p.dim() < 2)]
    rest = [p for n, p in m2.named_parameters() if ("norm" in n or "emb" in n or p.dim() < 2)]
    o2 = torch.optim.AdamW([{"params": decay, "weight_decay": 0.1}, {"params": rest, "weight_decay": 0.0}], lr=1e-2,
                           betas=(0.9, 0.95))
    ids = torch.randint(0, 512, (2, 64), device="cuda")
    for _ in range(3):
        m1(ids, labels=ids)["loss"].backward()
        o1.step()
        o1.zero_grad()
        m2(ids, labels=ids)["loss"].backward()
        torch.nn.utils.clip_grad_norm_(m2.parameters(), 1.0)
        o2.step()
        o2.zero_grad()
    for (n, p), q in zip(m1.named_parameters(), m2.parameters()):
        assert torch.allclose(p, q, atol=3e-5), n


def test_bounded_wait_reports_instead_of_hanging():
    """A flag that nothing sets: the combine kernel gives up after its (short) budget, returns, and
    the host reads the status; the context stays usable."""
    import ctypes as C

    from nanopysche_b200.ops import _lib

    T, K, D = 8, 2, 256
    a = _lib.CombineArgs()
    rows = torch.zeros(T * K, D, device="cuda", dtype=torch.bfloat16)
    slot = torch.zeros(T, K, device="cuda", dtype=torch.int32)
    out = torch.zeros(T, D, device="cuda", dtype=torch.bfloat16)
    flags = torch.zeros(1, device="cuda", dtype=torch.int32)
    sent = torch.ones(1, device="cuda", dtype=torch.int32)
    a.rows, a.slot_pos, a.out = rows.data_ptr(), slot.data_ptr(), out.data_ptr()
    a.T, a.K, a.D, a.E = T, K, D, 1
    a.flags, a.sent_to_peer, a.n_ranks, a.epoch, a.limit_ns = flags.data_ptr(), sent.data_ptr(), 1, 5, 200_000_000
    _lib.check(_lib.lib().np_ep_combine(C.byref(a), C.c_void_p(_lib.stream())), "ep_combine")
    torch.cuda.synchronize()
    st = _lib.status()
    assert st[0] == 2 and st[1] == 11  # flag wait timed out, in the combine kernel
    _lib.lib().np_status_clear()
    assert (torch.ones(4, device="cuda") * 2).sum().item() == 8.0


def test_trainer_surfaces_a_timed_out_device_wait(tmp_path):
    """The same flag that nothing sets, launched from a callback in the middle of ``Trainer.fit()``: the trainer reads
    the status word at its next metric flush and raises ``CommTimeoutError`` (emergency checkpoint written)."""
    import ctypes as C

    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.engine import prepare_training
    from nanopysche_b200.fault_tolerance.hang_detection import CommTimeoutError
    from nanopysche_b200.ops import _lib
    from nanopysche_b200.train.callbacks.base import Callback
    from nanopysche_b200.train.trainer import Trainer, TrainingConfig

    torch.manual_seed(0)
    cfg = TransformerConfig(vocab_size=512, d_model=256, n_layers=1, n_heads=2, n_kv_heads=2, ffn_hidden=512,
                            max_seq_len=128, qk_norm=False)
    model = cfg.build(dtype=torch.bfloat16, init_device="cuda")
    opt, _ = prepare_training(model, tokens_per_rank=2 * 128, lr=1e-3)
    keep = []

    class StuckPeer(Callback):
        def post_step(self, t):
            if t.step != 2:
                return
            T, K, D = 8, 2, 256
            a = _lib.CombineArgs()
            bufs = [torch.zeros(T * K, D, device="cuda", dtype=torch.bfloat16),
                    torch.zeros(T, K, device="cuda", dtype=torch.int32),
                    torch.zeros(T, D, device="cuda", dtype=torch.bfloat16),
                    torch.zeros(1, device="cuda", dtype=torch.int32), torch.ones(1, device="cuda", dtype=torch.int32)]
            keep.extend(bufs)
            a.rows, a.slot_pos, a.out = bufs[0].data_ptr(), bufs[1].data_ptr(), bufs[2].data_ptr()
            a.T, a.K, a.D, a.E = T, K, D, 1
            a.flags, a.sent_to_peer, a.n_ranks, a.epoch, a.limit_ns = bufs[3].data_ptr(), bufs[4].data_ptr(), 1, 5, \
                200_000_000
            _lib.check(_lib.lib().np_ep_combine(C.byref(a), C.c_void_p(_lib.stream())), "ep_combine")

    tc = TrainingConfig(global_batch_size=2 * 128, micro_batch_size=2, sequence_length=128, max_steps=6,
                        log_interval=1, save_interval=0, save_dir=str(tmp_path), vocab_size=512)
    tr = Trainer(tc, model, opt, None, None, [StuckPeer()])
    with pytest.raises(CommTimeoutError):
        tr.fit()
    assert tr.step == 2 and tr.emergency_checkpoint_dir is not None
    assert (torch.ones(4, device="cuda") * 2).sum().item() == 8.0   # the context is still usable


def test_fused_moe_fp8_flow_path():
    """FP8-Flow-MoE recipe on the fused path: e4m3 dispatch + block-scaled fp8 expert GEMMs in forward,
    bf16 gradients; compared with the fp32 generic layer at fp8 tolerance."""
    from nanopysche_b200.models.moe import MoEBase
    from nanopysche_b200.ops.moe import build_runtime

    torch.manual_seed(0)
    B, S, D, H, E, K = 2, 256, 256, 256, 4, 2
    fused = MoEBase(d_model=D, hidden_size=H, num_experts=E, top_k=K, capacity_factor=1.25, dtype=torch.bfloat16,
                    device="cuda", init_std=0.05)
    ref = copy.deepcopy(fused).float()
    fused.fp8_flow_moe_enabled, fused.fp8_recipe, fused.fp8_gemm_threshold = True, "flow_moe", 64
    rt = build_runtime([fused], tokens=B * S, device=torch.device("cuda"))
    assert rt.fp8
    x = torch.randn(B, S, D, device="cuda").bfloat16()
    xa = x.clone().requires_grad_(True)
    y = fused(xa)
    gy = torch.randn_like(y)
    (y * gy).sum().backward()
    xb = x.float().requires_grad_(True)
    yr = ref(xb)
    (yr * gy.float()).sum().backward()
    assert rel(y, yr) < 0.08 and rel(xa.grad, xb.grad) < 0.08
    for n in ("w1", "w2", "w3"):
        assert rel(getattr(fused, n).grad, getattr(ref, n).grad) < 0.08, n


def test_moe_layer_mxfp8_recipe_on_gpu():
    """``mxfp8`` recipe with the fused runtime present: the layer leaves the fused path for the modular one whose
    expert GEMMs run on the block-scaled tcgen05 kernel (forward MXFP8, backward bf16)."""
    from nanopysche_b200.models.moe import MoEBase
    from nanopysche_b200.ops import _lib
    from nanopysche_b200.ops.moe import build_runtime

    torch.manual_seed(1)
    B, S, D, H, E, K = 2, 256, 256, 256, 4, 2
    moe = MoEBase(d_model=D, hidden_size=H, num_experts=E, top_k=K, dtype=torch.bfloat16, device="cuda", init_std=0.05,
                  fp8_flow_moe=True, fp8_recipe="mxfp8", fp8_gemm_threshold=64)
    ref = MoEBase(d_model=D, hidden_size=H, num_experts=E, top_k=K, dtype=torch.float32, device="cuda", init_std=0.05)
    ref.load_state_dict({k: v.float() for k, v in moe.state_dict().items()})
    build_runtime([moe], tokens=B * S, device=torch.device("cuda"))
    x = torch.randn(B, S, D, device="cuda").bfloat16()
    assert not moe._can_fuse(x)
    xa = x.clone().requires_grad_(True)
    y = moe(xa)
    assert moe._fp8_flow_moe.last_path == "mxfp8"
    gy = torch.randn_like(y)
    (y * gy).sum().backward()
    xb = x.float().requires_grad_(True)
    yr = ref(xb)
    (yr * gy.float()).sum().backward()
    _lib.check_status("mxfp8 moe")
    assert rel(y, yr) < 0.08 and rel(xa.grad, xb.grad) < 0.08
    for n in ("w1", "w2", "w3"):
        assert rel(getattr(moe, n).grad, getattr(ref, n).grad) < 0.08, n


def test_cli_train_and_bench_on_gpu(tmp_path, capsys):
    """The user-facing entry points on a GPU: a few optimizer steps of the 125m preset with MoE layers (12 heads of
    dim 64: attention runs on the flash kernels with the head dimension zero-padded to 128; fused-MoE and arena
    paths) and the forward benchmark, through ``cli.main``."""
    from nanopysche_b200 import cli
    from nanopysche_b200.ops import _lib

    args = ["--model", "125m", "--use-moe", "--num-experts", "4", "--top-k", "2", "--batch-size", "2", "--seq-len", "256",
            "--device", "cuda"]
    l0 = _lib.LAUNCHES
    rc = cli.main(["train", *args, "--max-steps", "3", "--save-dir", str(tmp_path / "ck"), "--log-interval", "1"])
    assert rc in (0, None)
    assert _lib.LAUNCHES > l0, "the CUDA kernels were not used"
    _lib.check_status("cli train")
    rc = cli.main(["bench", *args, "--warmup", "1", "--iters", "2"])
    assert rc in (0, None)
    out = capsys.readouterr().out
    assert "tokens/s" in out or "tok/s" in out.lower()


def test_checkpoint_round_trip_on_gpu_with_equal_layer_shapes(tmp_path):
    """Pinned staging must not alias tensors of equal shape and dtype: save a three-layer model whose layers all
    have the same shapes from the GPU, load it into a fresh model, compare every tensor."""
    from nanopysche_b200.checkpoint.distributed import CheckpointConfig, DistributedCheckpointer
    from nanopysche_b200.config import TransformerConfig

    def build(seed):
        torch.manual_seed(seed)
        cfg = TransformerConfig(vocab_size=256, d_model=128, n_layers=3, n_heads=2, n_kv_heads=2, ffn_hidden=256,
                                max_seq_len=64, qk_norm=False)
        return cfg.build(dtype=torch.bfloat16, init_device="cuda")

    m = build(0)
    with torch.no_grad():
        for i, blk in enumerate(m.blocks.values()):
            blk.attention.w_q.weight.fill_(float(i + 1))
    ck = DistributedCheckpointer(CheckpointConfig(save_dir=str(tmp_path), pinned_memory=True))
    assert ck.stager.enabled
    ck.save(3, m)
    m2 = build(1)
    ck.load(model=m2)
    for k, v in m.state_dict().items():
        assert torch.equal(m2.state_dict()[k], v), k


def test_same_seed_gives_the_same_first_loss_bit_for_bit_and_the_same_trajectory():
    """Determinism: forward pass and loss have a fixed reduction order, so two runs from one seed agree bit for bit on
    the first loss; the following steps go through gradients accumulated with atomics (embedding rows, router
    statistics) and agree to rounding."""
    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.engine import prepare_training

    def run():
        torch.manual_seed(11)
        cfg = TransformerConfig(vocab_size=1024, d_model=256, n_layers=2, n_heads=2, n_kv_heads=1, ffn_hidden=512,
                                rope_base=10000.0, max_seq_len=256, qk_norm=False, use_moe=True, num_experts=4,
                                moe_top_k=2, moe_interval=1, moe_hidden=256, moe_capacity_factor=1.25)
        model = cfg.build(dtype=torch.bfloat16, init_device="cuda")
        opt, _ = prepare_training(model, tokens_per_rank=2 * 256, lr=1e-3)
        ids = torch.randint(0, 1024, (2, 256), device="cuda")
        out = []
        for _ in range(4):
            o = model(ids, labels=ids)
            (o["loss"] + o["aux_loss"]).backward()
            opt.step()
            opt.zero_grad()
            out.append(o["loss"].item())
        return out

    a, b = run(), run()
    assert a[0] == b[0], (a, b)
    for x, y in zip(a, b):
        assert abs(x - y) <= 2e-3 * abs(x), (a, b)
