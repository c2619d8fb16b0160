"""fp8_flow_moe package: operator semantics on CPU, kernel parity on GPU."""
import pytest
import torch
import torch.nn.functional as F

import fp8_flow_moe as fm
from fp8_flow_moe import ops


def test_public_names_and_recipes():
    for n in ("FP8FlowMoEConfig", "FP8FlowMoECompute", "FP8RecipeConfig", "FP8RecipeType", "BlockScalingGranularity",
              "quantize_to_fp8", "dequantize_from_fp8", "scaling_aware_transpose", "fused_swiglu_quantize",
              "fused_silu_multiply_quantize", "fused_permute_pad", "fused_unpermute_unpad", "fp8_grouped_gemm"):
        assert hasattr(fm, n), n
    assert fm.FP8_BLOCK_SIZE == 128
    assert [t.value for t in fm.FP8RecipeType] == ["none", "blockwise", "mxfp8", "flow_moe"]
    assert fm.FP8RecipeConfig(True, "mxfp8").block_size == 32 and not fm.FP8RecipeConfig(True, "none").active
    import nanopysche_b200.fp8 as nf

    assert nf.FP8FlowMoECompute is fm.FP8FlowMoECompute and nf.FP8_BLOCK_SIZE == 128


def test_quant_dequant_roundtrip_and_scales():
    torch.manual_seed(0)
    x = torch.randn(6, 384) * torch.logspace(-2, 2, 6).unsqueeze(1)
    q, s = ops.quantize_to_fp8(x)
    assert q.dtype == torch.float8_e4m3fn and s.shape == (6, 3)
    assert torch.allclose(s, x.reshape(6, 3, 128).abs().amax(-1) / 448.0)
    back = ops.dequantize_from_fp8(q, s, dtype=torch.float32)
    assert ((back - x).abs() <= x.reshape(6, 3, 128).abs().amax(-1).repeat_interleave(128, 1) * 0.0626).all()
    q2, s2 = ops.quantize_to_fp8(x, block_size=32, pow2_scales=True)
    assert s2.shape == (6, 12) and torch.equal(torch.log2(s2), torch.log2(s2).round())
    wq, ws = ops.quantize_weight_blockwise(torch.randn(256, 384))
    assert ws.shape == (2, 3) and ops.dequantize_from_fp8(wq, ws, dtype=torch.float32).shape == (256, 384)


def test_scaling_aware_transpose():
    torch.manual_seed(1)
    x = torch.randn(256, 384)
    q, s = ops.quantize_to_fp8(x)
    qt, st = ops.scaling_aware_transpose(q, s)
    assert qt.shape == (384, 256) and st.shape == (384, 2)
    ref = ops.dequantize_from_fp8(q, s, dtype=torch.float32).t()
    got = ops.dequantize_from_fp8(qt, st, dtype=torch.float32)
    assert ((got - ref).norm() / ref.norm()).item() < 0.04


def test_permute_pad_and_grouped_gemm():
    torch.manual_seed(2)
    n, D, E, N = 300, 128, 4, 256
    x = torch.randn(n, D)
    idx = torch.randint(0, E, (n,))
    xp, row_map, padded = ops.fused_permute_pad(x, idx, E, 128)
    assert (padded % 128 == 0).all() and xp.shape[0] == int(padded.sum())
    assert torch.equal(ops.fused_unpermute_unpad(xp, row_map), x)
    starts = torch.cumsum(padded, 0) - padded
    assert ((row_map >= starts[idx]) & (row_map < starts[idx] + padded[idx])).all()
    counts = torch.bincount(idx, minlength=E)
    for e in range(E):  # padding rows are zero
        assert xp[starts[e] + counts[e]: starts[e] + padded[e]].abs().sum() == 0
    w = torch.randn(E, N, D) * 0.1
    xq, xs = ops.quantize_to_fp8(xp)
    wq, ws = ops.quantize_weight_blockwise(w.reshape(E * N, D))
    y = ops.fp8_grouped_gemm(xq, xs, wq.view(E, N, D), ws.view(E, N // 128, D // 128), padded, out_dtype=torch.float32)
    ref = torch.stack([x[i] @ w[idx[i]].t() for i in range(n)])
    got = ops.fused_unpermute_unpad(y, row_map)
    assert ((got - ref).norm() / ref.norm()).item() < 0.06
    wts = torch.rand(n)
    assert torch.allclose(ops.fused_unpermute_unpad(y, row_map, wts), got * wts[:, None])


def test_swiglu_quantize():
    g, u = torch.randn(4, 256), torch.randn(4, 256)
    q, s = ops.fused_silu_multiply_quantize(g, u)
    ref = F.silu(g) * u
    assert ((ops.dequantize_from_fp8(q, s, dtype=torch.float32) - ref).norm() / ref.norm()).item() < 0.04
    q2, s2 = ops.fused_swiglu_quantize(torch.cat([g, u], -1))
    assert torch.equal(q.float(), q2.float()) and torch.equal(s, s2)


def test_flow_moe_compute_threshold_switch_and_grads():
    torch.manual_seed(3)
    E, H, D = 2, 128, 128
    w1, w2, w3 = (torch.nn.Parameter(torch.randn(E * H, D) * 0.1) for _ in range(3))
    cfg = fm.FP8FlowMoEConfig(True, fm.FP8RecipeConfig(True, "flow_moe"))
    comp = fm.FP8FlowMoECompute(cfg, D, H, E, fp8_gemm_threshold=64)
    comp.set_weights(w1, w2, w3)
    x = torch.randn(400, D, requires_grad=True)
    idx = torch.randint(0, E, (400,))
    y = comp(x, None, idx, 0, E)
    assert comp.last_path == "fp8"
    ref = torch.stack([(F.silu(x[i] @ w1[idx[i] * H:(idx[i] + 1) * H].t()) * (x[i] @ w3[idx[i] * H:(idx[i] + 1) * H].t()))
                       @ w2[idx[i] * H:(idx[i] + 1) * H] for i in range(400)])
    assert ((y - ref).norm() / ref.norm()).item() < 0.08
    y.sum().backward()
    assert x.grad is not None and w1.grad is not None
    small = comp(x[:20].detach(), None, idx[:20], 0, E)
    assert comp.last_path == "bf16" and torch.allclose(small, ref[:20], atol=1e-4)
    off = fm.FP8FlowMoECompute(fm.FP8FlowMoEConfig(False), D, H, E, fp8_gemm_threshold=1)
    off.set_weights(w1, w2, w3)
    off(x.detach(), None, idx, 0, E)
    assert off.last_path == "bf16"


def test_flow_moe_compute_mxfp8_recipe():
    """1x32 power-of-two scaled expert GEMMs (grouped form) against the per-row fp32 expert MLP."""
    torch.manual_seed(5)
    E, H, D = 3, 128, 256
    w1, w2, w3 = (torch.nn.Parameter(torch.randn(E * H, D) * 0.1) for _ in range(3))
    comp = fm.FP8FlowMoECompute(fm.FP8FlowMoEConfig(True, fm.FP8RecipeConfig(True, "mxfp8")), D, H, E,
                                fp8_gemm_threshold=16)
    assert comp.config.fp8_recipe.block_size == 32
    comp.set_weights(w1, w2, w3)
    x = torch.randn(300, D, requires_grad=True)
    idx = torch.randint(0, E, (300,))
    wts = torch.rand(300)
    y = comp(x, wts, idx, 0, E)
    assert comp.last_path == "mxfp8"
    ref = torch.stack([(F.silu(x[i] @ w1[idx[i] * H:(idx[i] + 1) * H].t()) * (x[i] @ w3[idx[i] * H:(idx[i] + 1) * H].t()))
                       @ w2[idx[i] * H:(idx[i] + 1) * H] for i in range(300)]) * wts.view(-1, 1)
    assert ((y - ref).norm() / ref.norm()).item() < 0.08
    gy = torch.randn_like(y)
    y.backward(gy)
    got = [t.grad.clone() for t in (x, w1, w2, w3)]
    for t in (x, w1, w2, w3):
        t.grad = None
    ref.backward(gy)
    for a, t, name in zip(got, (x, w1, w2, w3), ("x", "w1", "w2", "w3")):   # bf16 backward on the saved fp8 forward
        assert ((a - t.grad).norm() / t.grad.norm()).item() < 0.08, name


def test_moe_layer_with_flow_moe_recipe_and_fp8_linear():
    from nanopysche_b200.fp8.training import FP8Config, Float8Linear, apply_fp8, precompute_fp8_dynamic_scales
    from nanopysche_b200.models.moe import MoEBase

    torch.manual_seed(4)
    m = MoEBase(d_model=128, hidden_size=256, num_experts=2, top_k=1, fp8_flow_moe=True, fp8_recipe="flow_moe",
                fp8_gemm_threshold=8)
    ref = MoEBase(d_model=128, hidden_size=256, num_experts=2, top_k=1)
    ref.load_state_dict(m.state_dict())
    x = torch.randn(2, 64, 128)
    y, yr = m(x), ref(x)
    assert m._fp8_flow_moe.last_path == "fp8" and ((y - yr).norm() / yr.norm()).item() < 0.1
    net = torch.nn.Sequential(torch.nn.Linear(128, 256), torch.nn.ReLU(), torch.nn.Linear(256, 128))
    full = net(x).detach()
    apply_fp8(net, FP8Config(enabled=True))
    assert isinstance(net[0], Float8Linear) and precompute_fp8_dynamic_scales(net) == 2
    out = net(x)
    out.sum().backward()
    assert ((out - full).norm() / full.norm()).item() < 0.1 and net[0].weight.grad is not None
    assert net[0].weight._fp8_recipe == "blockwise"
    net_mx = torch.nn.Sequential(torch.nn.Linear(128, 256), torch.nn.ReLU(), torch.nn.Linear(256, 128))
    net_mx.load_state_dict({k: v for k, v in net.state_dict().items()})
    apply_fp8(net_mx, FP8Config(enabled=True, recipe_name="mxfp8"))
    assert net_mx[2].weight._fp8_recipe == "mxfp8"
    out_mx = net_mx(x)
    out_mx.sum().backward()
    assert ((out_mx - full).norm() / full.norm()).item() < 0.1 and net_mx[2].weight.grad is not None
    assert not torch.equal(out_mx, out)


@pytest.mark.gpu
def test_fp8_kernels_match_torch_reference():
    torch.manual_seed(5)
    x = (torch.randn(512, 1024, device="cuda") * 3).bfloat16()
    q, s = ops.quantize_to_fp8(x)
    xb = x.float().reshape(512, 8, 128)
    s_ref = xb.abs().amax(-1) / 448.0
    assert torch.allclose(s, s_ref, rtol=1e-6)
    q_ref = (xb / s_ref.unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn).reshape(512, 1024)
    assert (q.float() != q_ref.float()).float().mean() < 1e-3
    d = ops.dequantize_from_fp8(q, s)
    assert ((d.float() - x.float()).norm() / x.float().norm()).item() < 0.04
    wq, ws = ops.quantize_weight_blockwise(x)
    assert torch.allclose(ws, x.float().reshape(4, 128, 8, 128).abs().amax((1, 3)) / 448.0, rtol=1e-6)
    qt, st = ops.scaling_aware_transpose(q, s)
    ref_t = ops.dequantize_from_fp8(q, s, dtype=torch.float32).t()
    got_t = ops.dequantize_from_fp8(qt, st, dtype=torch.float32)
    assert ((got_t - ref_t).norm() / ref_t.norm()).item() < 0.04
    g, u = torch.randn(256, 512, device="cuda").bfloat16(), torch.randn(256, 512, device="cuda").bfloat16()
    hq, hs = ops.fused_silu_multiply_quantize(g, u)
    ref = F.silu(g.float()) * u.float()
    assert ((ops.dequantize_from_fp8(hq, hs, dtype=torch.float32) - ref).norm() / ref.norm()).item() < 0.04


def test_rmsnorm_with_fp8_output_cpu_path():
    from nanopysche_b200.ops.norm import rms_norm_quant, rms_norm_ref

    torch.manual_seed(6)
    x, res, w = torch.randn(10, 256), torch.randn(10, 256), torch.rand(256) + 0.5
    q, s, h, y = rms_norm_quant(x, w, 1e-6, res, return_bf16=True)
    y_ref, h_ref = rms_norm_ref(x, w, 1e-6, res)
    assert torch.equal(h, h_ref) and torch.equal(y, y_ref) and q.shape == (10, 256) and s.shape == (10, 2)
    assert ((ops.dequantize_from_fp8(q, s, dtype=torch.float32) - y_ref).norm() / y_ref.norm()).item() < 0.04


@pytest.mark.gpu
def test_permute_pad_kernels_match_the_sorting_statement_and_differentiate():
    """``fused_permute_pad`` / ``fused_unpermute_unpad`` on the GPU (counting-sort positions + row kernels) against the
    argsort statement of the same functions on CPU tensors, values and gradients."""
    torch.manual_seed(3)
    n, D, E = 777, 256, 5
    x = torch.randn(n, D, device="cuda").bfloat16()
    idx = torch.randint(0, E, (n,), device="cuda")
    idx[idx == 3] = 2                                    # an expert with no rows
    w = torch.rand(n, device="cuda")
    xa = x.clone().requires_grad_(True)
    wa = w.clone().requires_grad_(True)
    out, row_map, padded = ops.fused_permute_pad(xa, idx, E, 128)
    back = ops.fused_unpermute_unpad(out * 2.0, row_map, wa)
    back.float().pow(2).sum().backward()
    xc = x.cpu().float().requires_grad_(True)
    wc = w.cpu().clone().requires_grad_(True)
    out_c, map_c, pad_c = ops.fused_permute_pad(xc, idx.cpu(), E, 128)
    back_c = ops.fused_unpermute_unpad(out_c * 2.0, map_c, wc)
    back_c.pow(2).sum().backward()
    assert torch.equal(row_map.cpu(), map_c) and torch.equal(padded.cpu(), pad_c)
    assert torch.equal(out.float().cpu(), out_c.detach().bfloat16().float())
    assert ((back.float().cpu() - back_c.detach()).norm() / back_c.detach().norm()).item() < 1e-2
    assert ((xa.grad.float().cpu() - xc.grad).norm() / xc.grad.norm()).item() < 2e-2
    assert ((wa.grad.cpu() - wc.grad).norm() / wc.grad.norm()).item() < 2e-2
