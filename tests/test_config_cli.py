"""Config system, presets, CLI parser, schedulers, bench utils (CPU)."""
import json
import math

import pytest
import torch

from nanopysche_b200 import bench_utils
from nanopysche_b200.cli import MODEL_PRESETS, build_parser, main
from nanopysche_b200.config import ExperimentConfig, TrainingConfig, TransformerConfig
from nanopysche_b200.train.scheduler import (CosineWithWarmup, WarmupStableDecay, cosine_with_warmup,
                                             exponential_decay, warmup_stable_decay)


def test_config_roundtrip_json_yaml_toml(tmp_path):
    cfg = ExperimentConfig(name="x", model=TransformerConfig(d_model=128, n_layers=3), seed=7)
    for ext in ("json", "yaml"):
        p = tmp_path / f"c.{ext}"
        cfg.save(p)
        back = ExperimentConfig.load(p)
        assert back.model.d_model == 128 and back.model.n_layers == 3 and back.seed == 7
        assert isinstance(back.model, TransformerConfig)


def test_merge_and_from_cli():
    cfg = ExperimentConfig().merge({"model.d_model": 256, "training.learning_rate": 1e-3, "nope.x": 1})
    assert cfg.model.d_model == 256 and cfg.training.learning_rate == 1e-3
    t = TransformerConfig.from_cli(["--d_model", "512", "--qk_norm", "false", "--ffn_hidden", "none",
                                    "--rope_base", "1e4"])
    assert t.d_model == 512 and t.qk_norm is False and t.ffn_hidden is None and t.rope_base == 1e4


def test_transformer_config_build_defaults():
    m = TransformerConfig(d_model=96, n_layers=2, n_heads=4, vocab_size=50, max_seq_len=16).build()
    ff = m.blocks["0"].feed_forward
    assert ff.hidden_size == 256  # int(8/3*96)=256 rounded up to 256
    assert m.blocks["0"].attention.q_norm is not None  # qk_norm defaults on
    assert "blocks.1.feed_forward.w2.weight" in m.state_dict()


def test_training_config_build_keeps_log_interval():
    tc = TrainingConfig(log_interval=3, global_batch_size=64, micro_batch_size=2, sequence_length=8).build()
    assert tc.log_interval == 3 and tc.dtype == torch.bfloat16
    assert tc.gradient_accumulation_steps == 4


def test_accumulation_never_zero():
    from nanopysche_b200.train.trainer import TrainingConfig as TC

    assert TC(global_batch_size=4, micro_batch_size=4, sequence_length=2048).gradient_accumulation_steps == 1
    assert TC(global_batch_size=4 * 2048 * 8, micro_batch_size=4, sequence_length=2048,
              dp_world_size=2).gradient_accumulation_steps == 4


def test_experiment_build():
    cfg = ExperimentConfig(model=TransformerConfig(d_model=64, n_layers=1, n_heads=2, vocab_size=40, max_seq_len=8),
                           training=TrainingConfig(warmup_steps=2, max_steps=10))
    model, opt, sched, tc = cfg.build()
    assert isinstance(sched, CosineWithWarmup) and opt.param_groups[0]["betas"] == (0.9, 0.95)


def test_presets_and_parser():
    assert MODEL_PRESETS["125m"] == dict(d_model=768, n_layers=12, n_heads=12, n_kv_heads=12, ffn_hidden=2048)
    assert MODEL_PRESETS["7b"]["ffn_hidden"] == 11008 and MODEL_PRESETS["1b"]["n_heads"] == 32
    p = build_parser()
    a = p.parse_args(["train", "--model", "350m", "--use-moe", "--num-experts", "4", "--top-k", "1", "--fp8-recipe",
                      "flow_moe", "--tp-size", "2", "--fsdp", "--ac-mode", "full", "--resume", "x", "--wandb"])
    assert a.command == "train" and a.use_moe and a.num_experts == 4 and a.fp8_recipe == "flow_moe" and a.fsdp
    b = p.parse_args(["bench", "--warmup", "1", "--iters", "2", "--validate"])
    assert b.fp8_gemm_threshold == 1000000 and b.iters == 2 and b.validate


def test_schedules():
    assert cosine_with_warmup(0, 10, 100, 0.1, 1.0) == 0.0
    assert cosine_with_warmup(10, 10, 100, 0.1, 1.0) == pytest.approx(1.0)
    assert cosine_with_warmup(55, 10, 100, 0.1, 1.0) == pytest.approx(0.1 + 0.45 * (1 + math.cos(math.pi / 2)))
    assert cosine_with_warmup(500, 10, 100, 0.1, 1.0) == 0.1
    assert warmup_stable_decay(15, 10, 10, 10, 0.1, 1.0) == 1.0
    assert warmup_stable_decay(30, 10, 10, 10, 0.1, 1.0) == 0.1
    assert exponential_decay(12, 10, 0.5, 0.0, 1.0) == 0.25
    opt = torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=2.0)
    s = WarmupStableDecay(opt, 2, 2, 4, 0.1)
    lrs = []
    for _ in range(9):
        lrs.append(opt.param_groups[0]["lr"])
        opt.step()
        s.step()
    assert lrs[0] == 0.0 and lrs[2] == 2.0 and lrs[3] == 2.0 and lrs[8] == pytest.approx(0.2)


def test_bench_utils():
    f = bench_utils.estimate_model_flops(2, 64, 256, 4, 16, 2)
    per_tok = 2 * (8 * 64 * 64 + 4 * 16 * 64) + 2 * 6 * 64 * 256
    assert f == 3.0 * (per_tok * 32 + 2 * 64 * 32)
    moe = bench_utils.estimate_model_flops(2, 64, 256, 4, 16, 2, num_experts=8, top_k=2)
    assert moe > f
    assert bench_utils.PEAK_FLOPS["B200"] == 2250e12 and bench_utils.FP8_PEAK_FLOPS["B200"] == 4500e12
    mfu = bench_utils.compute_mfu(1.0, 2, 64, 256, 4, 16, 2)
    assert mfu > 0 if torch.cuda.is_available() else mfu == 0.0      # no peak to relate to on a CPU, as in the reference


def test_cli_bench_cpu(capsys):
    rc = main(["bench", "--model", "125m", "--batch-size", "1", "--seq-len", "16", "--device", "cpu", "--iters", "1",
               "--warmup", "0", "--forward-only"])
    assert rc == 0 and "tokens/s" in capsys.readouterr().out
