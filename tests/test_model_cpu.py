"""Model layer on CPU: op references, blocks, MoE semantics, the 125m config end to end."""
import copy
import math

import pytest
import torch
import torch.nn.functional as F

from nanopysche_b200.config import TransformerConfig
from nanopysche_b200.models import Attention, FeedForward, MoEBase, RMSNorm, RotaryEmbedding, Transformer
from nanopysche_b200.models.moe import MoERouter, MoERouterConfig, NcclAllToAllDispatcher
from nanopysche_b200.models.rope import RoPEScalingConfig, apply_rotary_emb
from nanopysche_b200.ops import attention as attn_ops
from nanopysche_b200.ops import rope as rope_ops


def test_rmsnorm_matches_formula_and_fused_residual():
    n = RMSNorm(32)
    with torch.no_grad():
        n.weight.uniform_(0.5, 1.5)
    x, r = torch.randn(3, 5, 32), torch.randn(3, 5, 32)
    ref = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-6) * n.weight
    assert torch.allclose(n(x), ref, atol=1e-6)
    y, h = n(x, residual=r)
    assert torch.allclose(h, x + r) and torch.allclose(y, n(x + r), atol=1e-6)
    n.to(torch.bfloat16)
    assert n.weight.dtype == torch.float32


def test_rope_matches_reference_formula():
    rot = RotaryEmbedding(16, base=10000.0, max_seq_len=32)
    cos, sin = rot(8, offset=2, device="cpu")
    inv = 1.0 / (10000.0 ** (torch.arange(0, 16, 2).float() / 16))
    ang = torch.outer(torch.arange(2, 10).float(), inv)
    assert torch.allclose(cos, torch.cat([ang, ang], -1).cos(), atol=1e-6)
    x = torch.randn(2, 8, 3, 16)
    ref = apply_rotary_emb(x, cos, sin, head_first=True)
    c, s = rot.half_tables(10, "cpu")
    got = rope_ops.apply_rope_ref(x, c, s, pos_offset=2)
    assert torch.allclose(got, ref, atol=1e-5)
    # inverse rotation undoes it
    back = rope_ops.apply_rope_ref(got, c, s, pos_offset=2, sign=-1.0)
    assert torch.allclose(back, x, atol=1e-5)


def test_rope_scaling_piecewise_and_yarn():
    sc = RoPEScalingConfig(factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                           original_max_position_embeddings=64)
    c1, _ = rope_ops.rope_tables_ref(4, 32, 10000.0, "piecewise", 8.0, 64.0, 1.0, 4.0)
    c0, _ = rope_ops.rope_tables_ref(4, 32, 10000.0)
    inv = 10000.0 ** (-torch.arange(16).float() * 2 / 32)
    wl = 2 * math.pi / inv
    exp_inv = torch.where(wl < 16.0, inv, torch.where(wl > 64.0, inv / 8.0, inv))
    assert torch.allclose(c1, torch.outer(torch.arange(4.0), exp_inv).cos(), atol=1e-6)
    assert not torch.allclose(c1, c0)
    cy, sy = rope_ops.rope_tables_ref(4, 32, 10000.0, "yarn", 8.0, 64.0, 1.0, 32.0)
    assert cy[0, 0] == pytest.approx(rope_ops.yarn_mscale(8.0))  # cos(0) * mscale
    r = RotaryEmbedding(32, scaling=sc)
    assert r.half_tables(4, "cpu")[0].shape[1] == 16


def test_attention_gqa_matches_expanded_sdpa_and_kv_cache():
    torch.manual_seed(0)
    a = Attention(d_model=64, n_heads=4, n_kv_heads=2, max_seq_len=32)
    x = torch.randn(2, 10, 64)
    y = a(x)
    # manual: expand kv heads like the reference does
    q = a.w_q(x).view(2, 10, 4, 16)
    k = a.w_k(x).view(2, 10, 2, 16)
    v = a.w_v(x).view(2, 10, 2, 16)
    cos, sin = a.rope(10, device="cpu")
    q, k = apply_rotary_emb(q, cos, sin), apply_rotary_emb(k, cos, sin)
    k, v = k.repeat_interleave(2, 2), v.repeat_interleave(2, 2)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True)
    ref = a.w_out(o.transpose(1, 2).reshape(2, 10, 64))
    assert torch.allclose(y, ref, atol=1e-5)
    # incremental decoding with a kv cache reproduces the full forward
    y1, kv = a(x[:, :6], return_kv=True)
    y2 = a(x[:, 6:], kv_cache=kv, start_pos=6)
    assert torch.allclose(torch.cat([y1, y2], 1), y, atol=1e-5)


def test_attention_ref_lse_and_merge():
    q, k, v = torch.randn(1, 6, 2, 8), torch.randn(1, 6, 2, 8), torch.randn(1, 6, 2, 8)
    full, lse = attn_ops.attention_ref(q, k, v, causal=False)
    o1, l1 = attn_ops.attention_ref(q, k[:, :2], v[:, :2], causal=False)
    o2, l2 = attn_ops.attention_ref(q, k[:, 2:], v[:, 2:], causal=False)
    m, lm = attn_ops.merge_attention(o1, l1, o2, l2)
    assert torch.allclose(m, full, atol=1e-5) and torch.allclose(lm, lse, atol=1e-5)
    # a fully masked query row yields zeros, not NaN
    o, l = attn_ops.attention_ref(q, k, v, causal=True, q_pos=torch.zeros(6, dtype=torch.long),
                                  k_pos=torch.arange(1, 7))
    assert torch.isfinite(o).all() and (o == 0).all() and torch.isinf(l).all()


def test_feed_forward_swiglu_geglu():
    f = FeedForward(d_model=32, hidden_size=64)
    x = torch.randn(4, 32)
    assert torch.allclose(f(x), f.w2(F.silu(f.w1(x)) * f.w3(x)), atol=1e-6)
    g = FeedForward(d_model=32, hidden_size=64, activation="gelu_tanh")
    assert torch.allclose(g(x), g.w2(F.gelu(g.w1(x), approximate="tanh") * g.w3(x)), atol=1e-6)
    assert FeedForward(d_model=96).hidden_size == 256


def test_router_softmax_sigmoid_aux_and_bias():
    torch.manual_seed(0)
    r = MoERouter(d_model=16, config=MoERouterConfig(num_experts=4, top_k=2, bias_gamma=0.1, z_loss_multiplier=0.01))
    assert torch.all(r.gate.bias == -1.0)
    x = torch.randn(2, 5, 16)
    w, idx, aux = r(x)
    logits = r.gate(x.float())
    tl, ti = logits.topk(2, -1)
    assert torch.equal(idx, ti) and torch.allclose(w, tl.softmax(-1), atol=1e-6)
    f = torch.bincount(idx.reshape(-1), minlength=4).float() / 10
    P = logits.softmax(-1).reshape(-1, 4).mean(0)
    exp = 4 * (f * P).sum() + 0.01 * torch.logsumexp(logits, -1).square().mean()
    assert aux.item() == pytest.approx(exp.item(), rel=1e-5)
    assert int(r._total_tokens_this_batch) == 20
    before = r.score_bias.clone()
    r.post_batch()
    load = f / 2
    assert torch.allclose(r.score_bias - before, -0.1 * (load - 0.25), atol=1e-6)  # over-loaded experts go down
    assert int(r._total_tokens_this_batch) == 0
    s = MoERouter(d_model=16, config=MoERouterConfig(num_experts=4, top_k=2, gating_function="sigmoid"))
    w2, _, _ = s(x)
    assert torch.allclose(w2.sum(-1), torch.ones(2, 5), atol=1e-5)


def test_routing_replay():
    r = MoERouter(d_model=8, config=MoERouterConfig(num_experts=4, top_k=1, routing_replay=True))
    x = torch.randn(1, 6, 8)
    mask = torch.zeros(1, 6, 4, dtype=torch.bool)
    mask[..., 3] = True
    r.set_replay_mask(mask)
    r.train()
    _, idx, _ = r(x)
    assert (idx == 3).all()
    r.clear_replay_mask()
    _, idx2, _ = r(x)
    assert torch.equal(idx2, r.gate(x).topk(1, -1).indices)


def _reference_capacity(indices, T, E, capacity):
    keep = torch.ones(T, dtype=torch.bool)
    drops = []
    for e in range(E):
        ids = (indices == e).any(-1).nonzero(as_tuple=True)[0]
        drops.append(max(0, len(ids) - capacity))
        if len(ids) > capacity:
            keep[ids[capacity:]] = False
    return keep, drops


def test_capacity_matches_reference_rule():
    torch.manual_seed(1)
    m = MoEBase(d_model=16, hidden_size=256, num_experts=4, top_k=2, capacity_factor=1.0)
    T = 40
    idx = torch.stack([torch.randperm(4)[:2] for _ in range(T)])
    x, w = torch.randn(T, 16), torch.rand(T, 2)
    xk, wk, ik, dropped, keep = m._apply_capacity(x, w, idx)
    ref_keep, ref_drops = _reference_capacity(idx, T, 4, int(1.0 * T / 4))
    assert torch.equal(keep, ref_keep) and m.per_expert_drops.tolist() == ref_drops
    assert m.last_dropped == int((~ref_keep).sum()) and m.total_tokens_routed == T
    assert xk.shape[0] == int(ref_keep.sum())
    st = m.get_drop_stats()
    assert st["drop_rate"] == pytest.approx(m.last_dropped / T) and st["capacity_factor"] == 1.0
    m.reset_drop_stats()
    assert m.total_dropped == 0


def test_moe_forward_equals_dense_loop_and_grads():
    torch.manual_seed(2)
    m = MoEBase(d_model=16, hidden_size=256, num_experts=4, top_k=2)
    x = torch.randn(2, 6, 16, requires_grad=True)
    y = m(x)
    w, idx, _ = m.router(x)
    xf = x.reshape(-1, 16)
    ref = torch.zeros_like(xf)
    H = m.hidden_size
    for t in range(xf.shape[0]):
        for k in range(2):
            e = int(idx.reshape(-1, 2)[t, k])
            w1, w2, w3 = m.w1[e * H:(e + 1) * H], m.w2[e * H:(e + 1) * H], m.w3[e * H:(e + 1) * H]
            ref[t] += w.reshape(-1, 2)[t, k] * ((F.silu(xf[t] @ w1.t()) * (xf[t] @ w3.t())) @ w2)
    assert torch.allclose(y.reshape(-1, 16), ref, atol=1e-5)
    (y.sum() + m.aux_loss).backward()
    assert m.w1.grad is not None and m.router.gate.weight.grad is not None and x.grad is not None


def test_moe_dropped_tokens_output_zero():
    torch.manual_seed(3)
    m = MoEBase(d_model=16, hidden_size=256, num_experts=2, top_k=1, capacity_factor=0.5)
    x = torch.randn(1, 16, 16)
    y = m(x)
    assert m.last_dropped > 0
    zero_rows = (y.reshape(-1, 16).abs().sum(-1) == 0).sum().item()
    assert zero_rows == m.last_dropped


def test_adaptive_capacity_moves():
    m = MoEBase(d_model=8, hidden_size=256, num_experts=4, top_k=1, capacity_factor=1.0, adaptive_capacity=True)
    idx = torch.zeros(64, 1, dtype=torch.long)  # everything to expert 0: heavy drops
    m._update_adaptive_capacity(64, idx)
    assert m.capacity_factor == pytest.approx(1.1) and m.adaptive_drop_rate_ema > 0


def test_dispatcher_single_rank_roundtrip():
    d = NcclAllToAllDispatcher()
    x = torch.randn(5, 4)
    idx = torch.tensor([[1, 0], [0, 2], [2, 1], [1, 2], [0, 1]])
    w = torch.rand(5, 2)
    rows, lw, li, meta = d.dispatch(x, idx, w, 3)
    assert torch.equal(li, torch.sort(idx.reshape(-1), stable=True).values)
    out = d.combine(rows, meta, x, w, idx)
    assert torch.allclose(out, x * w.sum(-1, keepdim=True), atol=1e-6)


def test_hybrid_block_and_moe_placement():
    cfg = TransformerConfig(d_model=32, n_layers=4, n_heads=2, vocab_size=50, max_seq_len=16, ffn_hidden=256,
                            use_moe=True, num_experts=4, moe_interval=2, moe_offset=1, moe_hidden=256,
                            moe_keep_dense_ffn=True, qk_norm=False)
    m = cfg.build()
    kinds = [type(b).__name__ for b in m.blocks.values()]
    assert kinds == ["TransformerBlock", "MoEHybridTransformerBlock"] * 2
    blk = m.blocks["1"]
    assert blk.dense_ffn is not None and blk.feed_forward is blk.moe
    sd = m.state_dict()
    for k in ("blocks.1.moe.w1", "blocks.1.moe.router.gate.bias", "blocks.1.moe_norm.weight",
              "blocks.1.dense_ffn.w1.weight", "blocks.0.feed_forward.w3.weight", "lm_head.weight"):
        assert k in sd
    x = torch.randint(0, 50, (2, 8))
    out = m(x, labels=x)
    h = m.embeddings(x)
    a = h + blk.attention(blk.attention_norm(h))
    exp = a + blk.dense_ffn(blk.dense_norm(a)) + blk.moe(blk.moe_norm(a))
    assert torch.allclose(blk(h), exp, atol=1e-5)
    assert out["aux_loss"] is not None and torch.isfinite(out["loss"])


def test_transformer_loss_contract_and_tied():
    torch.manual_seed(0)
    m = Transformer(d_model=32, vocab_size=64, n_layers=2, block=dict(n_heads=2, max_seq_len=16, ffn_hidden=256))
    x = torch.randint(0, 64, (2, 9))
    labels = x.clone()
    labels[0, 3] = -100
    out = m(x, labels=labels)
    ref = F.cross_entropy(out["logits"][:, :-1].reshape(-1, 64), labels[:, 1:].reshape(-1), ignore_index=-100)
    assert out["loss"].item() == pytest.approx(ref.item(), rel=1e-6)
    t = Transformer(d_model=32, vocab_size=64, n_layers=1, block=dict(n_heads=2, max_seq_len=16, ffn_hidden=256),
                    tie_word_embeddings=True)
    assert t.lm_head is None and t(x)["logits"].shape == (2, 9, 64)
    assert m.num_params - m.num_non_embedding_params == 64 * 32


def test_125m_cpu_ten_adamw_steps_loss_decreases():
    """The 125m preset (12 layers, d 768, 12 heads of 64) at reduced sequence length so it stays fast: fp32, AdamW 3e-4,
    loss must go down and the checkpoint must round-trip."""
    torch.manual_seed(0)
    m = TransformerConfig(**{"vocab_size": 32000, "d_model": 768, "n_layers": 12, "n_heads": 12, "ffn_hidden": 2048,
                             "max_seq_len": 64, "qk_norm": True}).build()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.02)
    g = torch.Generator().manual_seed(0)
    x = torch.randint(0, 32000, (2, 64), generator=g)
    opt = torch.optim.AdamW(m.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    losses = []
    for _ in range(10):
        out = m(x, labels=x)
        out["loss"].backward()
        opt.step()
        opt.zero_grad()
        losses.append(out["loss"].item())
    assert losses[-1] < losses[0] - 0.5 and all(math.isfinite(l) for l in losses)


def test_deepep_dispatcher_knobs_map_onto_the_fused_runtime_settings():
    """``DeepEPDispatcher(num_sms=, use_fp8_dispatch=, adaptive=)``: explicit SM budget, roofline budget from
    ``AdaptiveSMAllocator`` (communication share of the layer's time on a 148-SM part), none by default."""
    from nanopysche_b200.models.moe import DeepEPDispatcher, ExpertParallelConfig

    shapes = dict(tokens=4096, d_model=2048, hidden=2816, num_experts=8, top_k=2)
    assert DeepEPDispatcher().dispatch_ctas(**shapes) == 0
    assert DeepEPDispatcher(num_sms=24).dispatch_ctas(**shapes) == 24
    a = DeepEPDispatcher(adaptive=True).dispatch_ctas(**shapes)
    b = DeepEPDispatcher(adaptive=True).dispatch_ctas(**shapes, fp8=True)
    assert 4 <= b <= a <= 144      # e4m3 rows halve the bytes on the wire, so fewer SMs go to the dispatch
    cfg = ExpertParallelConfig(ep_size=1, dispatcher=DeepEPDispatcher(use_fp8_dispatch=True))
    assert cfg.dispatcher.use_fp8_dispatch and cfg.dispatcher.async_with_compute_stream


def test_generic_adapter_layer_helpers():
    import torch.nn as nn

    from nanopysche_b200.models.parallel_adapter import iter_layers, layer_count

    class M(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleDict({str(i): nn.Linear(2, 2 + i) for i in (0, 1, 2, 10, 9)})

    m = M()
    assert layer_count(m) == 5
    assert [l.out_features for l in iter_layers(m)] == [2, 3, 4, 11, 12]      # numeric order: 9 before 10
    assert layer_count(nn.Linear(2, 2)) == 0 and list(iter_layers(nn.Linear(2, 2))) == []


def test_routing_prefetcher_votes_with_recency_and_scores_itself():
    from nanopysche_b200.models.ep_runtime import AdaptiveSMAllocator, CoupledEPScheduler, RoutingPrefetcher

    pf = RoutingPrefetcher(num_experts=4, history_len=3, confidence_threshold=0.8)
    stable = torch.tensor([[[0, 1], [2, 3]]])                  # (B=1, S=2, K=2)
    assert pf.predict_next_layer(0, stable) is None and not pf.should_prefetch(0)
    pf.record_routing(0, stable)
    pf.record_routing(0, stable)
    pred, conf = pf.predict_next_layer(0, stable)
    assert pred.shape == (1, 2, 2) and bool(conf.all())        # the same experts every step: confident
    assert set(pred[0, 0].tolist()) <= {0, 1} and set(pred[0, 1].tolist()) <= {2, 3}
    moved = torch.tensor([[[3, 2], [2, 3]]])                   # token 0 changes its experts in the newest step
    pf.record_routing(0, moved)
    pred, conf = pf.predict_next_layer(0, moved)
    assert int(pred[0, 0, 0]) in (2, 3) and not bool(conf[0, 0]) and bool(conf[0, 1])    # the newest step outvotes
    pf.record_outcome(pred, moved)
    st = pf.get_stats()
    assert st["total_predictions"] == 2 and st["hits"] == 2 and st["history_depth"] == {0: 3}

    # the SM split balances transfer and GEMM time: more bytes per FLOP -> more SMs for the exchange
    narrow = AdaptiveSMAllocator().compute_optimal_sms(4096, 2048, 2816, 8, 2)
    wide = AdaptiveSMAllocator().compute_optimal_sms(4096, 2048, 128, 8, 2)
    assert 4 <= narrow < wide <= 144
    sched = CoupledEPScheduler(8, 2048, 128)
    even = sched.schedule(torch.full((8,), 512.0), 4096, 2)
    skew = CoupledEPScheduler(8, 2048, 128).schedule(torch.tensor([64.0, 960.0] * 4), 4096, 2)
    assert even.dispatch_mode == "fast" and skew.imbalance_coefficient > even.imbalance_coefficient
    assert skew.num_sms >= even.num_sms and skew.prefetch_confidence < even.prefetch_confidence


def test_chunked_head_and_loss_equal_the_full_logits_path():
    """``loss_chunk_rows``: head projection and cross-entropy over a few rows at a time give the loss and every
    gradient of the path that forms all logits - with a chunk that does not divide the row count, ignored labels,
    tied embeddings, a scaled loss, and under the parameter arena (head gradient accumulated chunk by chunk into
    the arena buffer)."""
    import copy

    from nanopysche_b200.config import TransformerConfig
    from nanopysche_b200.optim.arena import ParamArena

    for tied in (False, True):
        torch.manual_seed(0)
        cfg = TransformerConfig(vocab_size=96, d_model=32, n_layers=2, n_heads=2, max_seq_len=16, ffn_hidden=256,
                                qk_norm=False, tie_word_embeddings=tied, xent_chunk_rows=5)
        chunked = cfg.build()
        assert chunked.loss_chunk_rows == 5
        full = copy.deepcopy(chunked)
        full.loss_chunk_rows = 0
        ids = torch.randint(0, 96, (3, 9))
        labels = ids.clone()
        labels[0, 3:6] = -100
        a, b = chunked(ids, labels=labels), full(ids, labels=labels)
        assert a["logits"] is None and b["logits"] is not None
        assert torch.allclose(a["loss"], b["loss"], atol=1e-6)
        (a["loss"] * 0.37).backward()
        (b["loss"] * 0.37).backward()
        for (n, p), q in zip(chunked.named_parameters(), full.parameters()):
            assert torch.allclose(p.grad, q.grad, atol=1e-6), n
    # arena: gradients of both paths land in the flat buffers
    torch.manual_seed(1)
    cfg = TransformerConfig(vocab_size=96, d_model=32, n_layers=1, n_heads=2, max_seq_len=16, ffn_hidden=256,
                            qk_norm=False)
    m1 = cfg.build()
    m2 = copy.deepcopy(m1)
    m1.loss_chunk_rows = 4
    a1, a2 = ParamArena(m1), ParamArena(m2)
    ids = torch.randint(0, 96, (2, 7))
    m1(ids, labels=ids)["loss"].backward()
    m2(ids, labels=ids)["loss"].backward()
    a1.collect_stray_grads() if hasattr(a1, "collect_stray_grads") else None
    a2.collect_stray_grads() if hasattr(a2, "collect_stray_grads") else None
    g1, g2 = dict(a1.named_main_grads()), dict(a2.named_main_grads())
    for n in g1:
        assert torch.allclose(g1[n], g2[n], atol=1e-6), n


def test_token_dropping_benchmark_counts():
    """``benchmarks.token_dropping``: overflow slots are what is left after every expert has filled its capacity, a
    dropped token is counted once however many of its experts were full, more capacity drops less."""
    from benchmarks.token_dropping import run

    rows = run(2048, 8, 2, 5.0, "cpu")
    by_cf = {r["capacity_factor"]: r for r in rows}
    assert by_cf[1.0]["overflow_slots"] == 2048 * 2 - 8 * 256          # every expert is over capacity at cf 1
    assert all(r["tokens_dropped"] <= r["overflow_slots"] for r in rows)
    drops = [by_cf[c]["tokens_dropped"] for c in (1.0, 1.25, 1.5, 2.0, 4.0)]
    assert drops == sorted(drops, reverse=True) and by_cf["dropless"]["tokens_dropped"] == 0
