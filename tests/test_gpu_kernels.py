"""sm_100a kernel numerics against plain PyTorch fp32 references of the same op (GPU only)."""
import math

import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.fixture(autouse=True)
def _status_clean():
    from nanopysche_b200.ops import _lib

    yield
    torch.cuda.synchronize()
    _lib.check_status("after test")


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 320), (200, 264, 72), (4096, 2048, 2048),
                                   (384, 32000, 256)])
@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_forward_shapes(M, N, K, bn):
    from nanopysche_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    assert rel(gemm(a, b, bn=bn), ref) < 4e-3
    assert rel(gemm(a, b, bn=bn, out_dtype=torch.float32), ref) < 1e-5


@pytest.mark.parametrize("bn", [128, 256])
def test_gemm_dgrad_wgrad_layouts_and_accumulate(bn):
    from nanopysche_b200.ops.gemm import gemm

    torch.manual_seed(1)
    dy = torch.randn(512, 384, device="cuda").bfloat16()
    w = torch.randn(384, 640, device="cuda").bfloat16()
    x = torch.randn(512, 640, device="cuda").bfloat16()
    assert rel(gemm(dy, w, b_mn=True, bn=bn), dy.float() @ w.float()) < 4e-3
    ref_w = dy.float().t() @ x.float()
    assert rel(gemm(dy, x, a_mn=True, b_mn=True, bn=bn, out_dtype=torch.float32), ref_w) < 1e-5
    acc = torch.full((384, 640), 2.0, device="cuda")
    gemm(dy, x, a_mn=True, b_mn=True, out=acc, accumulate=True, bn=bn)
    assert rel(acc, ref_w + 2.0) < 1e-5
    at = torch.randn(256, 384, device="cuda").bfloat16()
    bb = torch.randn(512, 256, device="cuda").bfloat16()
    assert rel(gemm(at, bb, a_mn=True, bn=bn, alpha=0.5), 0.5 * at.float().t() @ bb.float().t()) < 4e-3
    # strided operands (views into a wider buffer)
    wide = torch.randn(512, 1024, device="cuda").bfloat16()
    assert rel(gemm(wide[:, 128:384], w[:, :256].contiguous()), wide[:, 128:384].float() @ w[:, :256].float().t()) < 4e-3


def test_gemm_swiglu_epilogue():
    from nanopysche_b200.ops.gemm import gemm_swiglu

    torch.manual_seed(2)
    x = torch.randn(512, 256, device="cuda").bfloat16()
    w1 = (torch.randn(384, 256, device="cuda") * 0.1).bfloat16()
    w3 = (torch.randn(384, 256, device="cuda") * 0.1).bfloat16()
    h, gu = gemm_swiglu(x, w1, w3)
    g, u = x.float() @ w1.float().t(), x.float() @ w3.float().t()
    assert rel(h, F.silu(g) * u) < 6e-3 and rel(gu, torch.cat([g, u], 1)) < 4e-3


def test_linear_autograd_matches_torch():
    from nanopysche_b200.ops.gemm import linear

    torch.manual_seed(3)
    x = torch.randn(4, 96, 256, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(512, 256, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    y = linear(x, w)
    gy = torch.randn_like(y)
    y.backward(gy)
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = F.linear(xr, wr)
    yr.backward(gy.float())
    assert rel(y, yr) < 4e-3 and rel(x.grad, xr.grad) < 4e-3 and rel(w.grad, wr.grad) < 4e-3
    # main_grad accumulation (the arena path): two backward passes add up in fp32
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.zeros(512, 256, device="cuda")
    for _ in range(2):
        linear(x.detach(), w2).backward(gy)
    assert w2.grad is None and rel(w2.main_grad, 2 * wr.grad) < 1e-3


@pytest.mark.parametrize("rows,cols", [(64, 256), (4096, 2048), (300, 1024), (5, 2048), (33, 4096), (7, 8192)])
def test_rmsnorm_fwd_bwd(rows, cols):
    from nanopysche_b200.ops.norm import rms_norm, rms_norm_ref

    torch.manual_seed(4)
    x = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_(True)
    r = torch.randn(rows, cols, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.rand(cols, device="cuda") + 0.5).requires_grad_(True)
    y, h = rms_norm(x, w, 1e-6, r)
    gy, gh = torch.randn_like(y), torch.randn_like(h)
    (y * gy + h * gh).sum().backward()
    xr, rr, wr = (t.detach().float().requires_grad_(True) for t in (x, r, w))
    yr, hr = rms_norm_ref(xr, wr, 1e-6, rr)
    (yr * gy.float() + hr * gh.float()).sum().backward()
    assert rel(y, yr) < 6e-3 and rel(h, hr) < 4e-3
    assert rel(x.grad, xr.grad) < 8e-3 and rel(r.grad, rr.grad) < 8e-3 and rel(w.grad, wr.grad) < 8e-3
    y1 = rms_norm(x.detach(), w.detach())
    assert rel(y1, rms_norm_ref(x.detach().float(), w.detach())) < 6e-3


@pytest.mark.parametrize("act", ["silu", "gelu_tanh"])
def test_glu_fwd_bwd(act):
    from nanopysche_b200.ops.activation import glu, glu_ref

    torch.manual_seed(5)
    gu = torch.randn(300, 2 * 512, device="cuda").bfloat16().requires_grad_(True)
    h = glu(gu, act)
    gh = torch.randn_like(h)
    h.backward(gh)
    gr = gu.detach().float().requires_grad_(True)
    hr = glu_ref(gr, act)
    hr.backward(gh.float())
    assert rel(h, hr) < 6e-3 and rel(gu.grad, gr.grad) < 8e-3


def test_rope_kernel_and_tables():
    from nanopysche_b200.ops import rope as R

    for scaling, kw in ((None, {}), ("piecewise", dict(factor=8.0, orig_len=64.0, low_f=1.0, high_f=4.0)),
                        ("yarn", dict(factor=4.0, orig_len=64.0, low_f=1.0, high_f=32.0))):
        c, s = R.rope_tables(256, 128, 10000.0, scaling, device="cuda", **kw)
        cr, sr = R.rope_tables_ref(256, 128, 10000.0, scaling, device="cuda", **kw)
        assert torch.allclose(c, cr, atol=2e-4) and torch.allclose(s, sr, atol=2e-4), scaling
    torch.manual_seed(6)
    cos, sin = R.rope_tables(64, 128, 10000.0, device="cuda")
    qkv = torch.randn(2, 32, (4 + 2 + 2) * 128, device="cuda").bfloat16().requires_grad_(True)
    q = qkv[..., :512].unflatten(-1, (4, 128))  # strided view into the fused buffer
    out = R.apply_rope(q, cos, sin, pos_offset=3)
    ref = R.apply_rope_ref(q.detach().float(), cos, sin, pos_offset=3)
    assert rel(out, ref) < 6e-3
    g = torch.randn_like(out)
    out.backward(g)
    gref = R.apply_rope_ref(g.float(), cos, sin, pos_offset=3, sign=-1.0)
    assert rel(qkv.grad[..., :512].unflatten(-1, (4, 128)), gref) < 6e-3 and qkv.grad[..., 512:].abs().sum() == 0
    pid = torch.randint(0, 64, (2, 32), device="cuda")
    assert rel(R.apply_rope(q.detach(), cos, sin, pos_ids=pid),
               R.apply_rope_ref(q.detach().float(), cos, sin, pos_ids=pid)) < 6e-3


def test_cross_entropy_fwd_bwd():
    from nanopysche_b200.ops.xent import cross_entropy

    torch.manual_seed(7)
    logits = (torch.randn(300, 32000, device="cuda") * 2).bfloat16().requires_grad_(True)
    labels = torch.randint(0, 32000, (300,), device="cuda")
    labels[::7] = -100
    loss = cross_entropy(logits, labels)
    (loss * 3.0).backward()
    lr = logits.detach().float().requires_grad_(True)
    ref = F.cross_entropy(lr, labels, ignore_index=-100)
    (ref * 3.0).backward()
    assert abs(loss.item() - ref.item()) < 2e-3 * abs(ref.item())
    assert rel(logits.grad, lr.grad) < 1e-2


def test_fused_adamw_and_clip():
    from nanopysche_b200.ops import _lib

    torch.manual_seed(8)
    n = 100003
    p = torch.randn(n, device="cuda")
    g = torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    w16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    pr = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([pr], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    parts = _lib.lib().np_sumsq_parts()
    partial = torch.zeros(parts, device="cuda")
    coef = torch.zeros(2, device="cuda")
    for step in (1, 2, 3):
        _lib.call("sumsq", g, _lib.LL(n), partial)
        _lib.call("clip_coef", partial, parts, None, 1.0, coef)
        _lib.call("adamw", p, g, m, v, w16, _lib.LL(n), 1e-2, 0.9, 0.95, 1e-8, 0.1, step, coef[:1], None)
        pr.grad = g.clone()
        nrm = torch.nn.utils.clip_grad_norm_([pr], 1.0)
        opt.step()
        assert abs(coef[1].item() - nrm.item()) < 1e-3 * nrm.item()
    assert torch.allclose(p, pr.detach(), atol=1e-5) and rel(w16, p) < 4e-3


def test_router_kernels_match_module_math():
    from nanopysche_b200.models.moe import MoERouter, MoERouterConfig

    for gating in ("softmax", "sigmoid"):
        torch.manual_seed(9)
        r = MoERouter(d_model=512, config=MoERouterConfig(num_experts=8, top_k=2, gating_function=gating,
                                                         bias_gamma=0.01, z_loss_multiplier=0.001)).cuda()
        with torch.no_grad():
            r.score_bias.uniform_(-0.1, 0.1)
        x = torch.randn(3, 200, 512, device="cuda").bfloat16().requires_grad_(True)
        w, idx, aux = r(x)  # kernel path
        gw = torch.randn_like(w)
        ((w * gw).sum() + 2.0 * aux).backward()
        gx, ggw, ggb = x.grad.clone(), r.gate.weight.grad.clone(), r.gate.bias.grad.clone()
        r.zero_grad()
        xr = x.detach().float().requires_grad_(True)
        wr, ir, ar = r(xr)  # fp32 input -> PyTorch path
        ((wr * gw).sum() + 2.0 * ar).backward()
        same = (idx == ir).all(-1)
        assert same.float().mean() > 0.99  # bf16 rounding can flip near-ties
        assert rel(w[same], wr[same]) < 5e-3 and abs(aux.item() - ar.item()) < 5e-3 * abs(ar.item())
        assert rel(ggw, r.gate.weight.grad) < 2e-2 and rel(ggb, r.gate.bias.grad) < 2e-2
        assert rel(gx.float()[same], xr.grad[same]) < 3e-2


def test_capacity_scan_matches_reference_rule():
    from nanopysche_b200.ops import _lib

    torch.manual_seed(10)
    T, E, K = 1000, 8, 2
    idx = torch.stack([torch.randperm(E)[:K] for _ in range(T)]).to(torch.int32).cuda()
    for cap in (int(1.25 * T / E), 50, -1):
        slot_pos = torch.empty(T, K, dtype=torch.int32, device="cuda")
        keep = torch.empty(T, dtype=torch.int32, device="cuda")
        ck = torch.empty(E, dtype=torch.int32, device="cuda")
        drops = torch.empty(E, dtype=torch.int32, device="cuda")
        nd = torch.empty(1, dtype=torch.int32, device="cuda")
        _lib.call("capacity_scan", idx, T, E, K, cap, slot_pos, keep, ck, drops, nd)
        ic = idx.cpu().long()
        ref_keep = torch.ones(T, dtype=torch.bool)
        ref_drops = []
        for e in range(E):
            ids = (ic == e).any(-1).nonzero(as_tuple=True)[0]
            over = len(ids) - cap if cap >= 0 else 0
            ref_drops.append(max(0, over))
            if cap >= 0 and len(ids) > cap:
                ref_keep[ids[cap:]] = False
        assert torch.equal(keep.cpu().bool(), ref_keep) and drops.cpu().tolist() == ref_drops
        assert nd.item() == int((~ref_keep).sum())
        sp = slot_pos.cpu()
        for e in range(E):
            rows = [(t, k) for t in range(T) for k in range(K) if ic[t, k] == e and ref_keep[t]]
            assert ck[e].item() == len(rows)
            assert [sp[t, k].item() for t, k in rows] == list(range(len(rows)))
        assert (sp[~ref_keep] == -1).all()


def test_qkv_rope_fused_split():
    from nanopysche_b200.ops import rope as R

    torch.manual_seed(11)
    hq, hkv, hd = 4, 2, 128
    cos, sin = R.rope_tables(64, hd, 10000.0, device="cuda")
    qkv = torch.randn(2, 32, (hq + 2 * hkv) * hd, device="cuda").bfloat16().requires_grad_(True)
    q, k, v = R.qkv_rope(qkv, cos, sin, hq, hkv, hd, 5)
    qs = qkv.detach().float()[..., : hq * hd].unflatten(-1, (hq, hd))
    ks = qkv.detach().float()[..., hq * hd:(hq + hkv) * hd].unflatten(-1, (hkv, hd))
    vs = qkv.detach()[..., (hq + hkv) * hd:].unflatten(-1, (hkv, hd))
    assert rel(q, R.apply_rope_ref(qs, cos, sin, 5)) < 6e-3 and rel(k, R.apply_rope_ref(ks, cos, sin, 5)) < 6e-3
    assert torch.equal(v, vs)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    g = qkv.grad
    assert rel(g[..., : hq * hd].unflatten(-1, (hq, hd)), R.apply_rope_ref(gq.float(), cos, sin, 5, sign=-1.0)) < 6e-3
    assert rel(g[..., hq * hd:(hq + hkv) * hd].unflatten(-1, (hkv, hd)),
               R.apply_rope_ref(gk.float(), cos, sin, 5, sign=-1.0)) < 6e-3
    assert torch.equal(g[..., (hq + hkv) * hd:].unflatten(-1, (hkv, hd)), gv)


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (512, 384, 640), (4096, 2816, 2048), (4096, 2048, 2816)])
def test_fp8_block_gemm_matches_dequantised_reference(M, N, K):
    from fp8_flow_moe import ops as fops
    from nanopysche_b200.ops.gemm_fp8 import gemm_fp8_block, gemm_fp8_block_ref

    torch.manual_seed(12)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    xq, xs = fops.quantize_to_fp8(x)
    wq, ws = fops.quantize_weight_blockwise(w)
    got = gemm_fp8_block(xq, xs, wq, ws, out_dtype=torch.float32)
    ref = gemm_fp8_block_ref(xq, xs, wq, ws, out_dtype=torch.float32)
    assert rel(got, ref) < 1e-4
    assert rel(got, x.float() @ w.float().t()) < 0.06  # fp8 quantisation error


def test_fp8_block_gemm_grouped():
    from fp8_flow_moe import ops as fops
    from nanopysche_b200.ops.gemm_fp8 import gemm_fp8_block, gemm_fp8_block_ref

    torch.manual_seed(13)
    E, N, K, blocks = 4, 256, 512, 10
    x = torch.randn(blocks * 128, K, device="cuda").bfloat16()
    w = (torch.randn(E * N, K, device="cuda") * 0.05).bfloat16()
    grp = torch.tensor([0, 0, 1, 3, 3, 3, 2, -1, 1, 0], dtype=torch.int32, device="cuda")
    rows = torch.where(grp >= 0, 128, 0).to(torch.int32)
    xq, xs = fops.quantize_to_fp8(x)
    wq, ws = fops.quantize_weight_blockwise(w)
    out = torch.zeros(blocks * 128, N, device="cuda", dtype=torch.float32)
    gemm_fp8_block(xq, xs, wq, ws, out=out, mblk_group=grp.clamp_min(0), mblk_rows=rows, rows_per_group=N)
    ref = gemm_fp8_block_ref(xq, xs, wq, ws, grp, N, torch.float32)
    assert rel(out, ref) < 1e-4


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (200, 256, 384), (4096, 2816, 2048)])
def test_mxfp8_quantiser_and_gemm(M, N, K):
    """1x32 e8m0-scaled e4m3: the quantiser against its PyTorch statement (bit exact) and the block-scaled tcgen05
    GEMM against the fp32 product of the dequantised operands; scales vary per row and per 32-block."""
    from nanopysche_b200.ops.gemm_mxfp8 import gemm_mxfp8, gemm_mxfp8_ref, mx_quantize, mx_quantize_ref

    torch.manual_seed(14)
    sc = lambda r: torch.exp2(torch.randint(-8, 9, (r, K // 32), device="cuda").float()).repeat_interleave(32, 1)
    x = (torch.randn(M, K, device="cuda") * sc(M)).bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05 * sc(N)).bfloat16()
    xq, xs = mx_quantize(x)
    wq, ws = mx_quantize(w)
    xq_r, xs_r = mx_quantize_ref(x)
    assert torch.equal(xq.view(torch.uint8), xq_r.view(torch.uint8)) and torch.equal(xs, xs_r)
    got = gemm_mxfp8(xq, xs, wq, ws, out_dtype=torch.float32)
    assert rel(got, gemm_mxfp8_ref(xq, xs, wq, ws, out_dtype=torch.float32)) < 1e-4
    assert rel(got, x.float() @ w.float().t()) < 0.06
    assert rel(gemm_mxfp8(xq, xs, wq, ws), got) < 5e-3  # bf16 output


def test_mxfp8_gemm_grouped_and_linear():
    from nanopysche_b200.ops.gemm_mxfp8 import gemm_mxfp8, gemm_mxfp8_ref, mx_linear, mx_quantize

    torch.manual_seed(15)
    E, N, K, blocks = 4, 256, 512, 6
    x = torch.randn(blocks * 128, K, device="cuda").bfloat16()
    w = (torch.randn(E * N, K, device="cuda") * 0.05).bfloat16()
    grp = torch.tensor([0, 3, 1, 3, 2, 1], dtype=torch.int32, device="cuda")
    rows = torch.tensor([128, 128, 77, 0, 128, 128], dtype=torch.int32, device="cuda")
    xq, xs = mx_quantize(x)
    wq, ws = mx_quantize(w)
    out = torch.zeros(blocks * 128, N, device="cuda", dtype=torch.float32)
    gemm_mxfp8(xq, xs, wq, ws, out=out, mblk_group=grp, mblk_rows=rows, rows_per_group=N)
    ref = gemm_mxfp8_ref(xq, xs, wq, ws, grp, N, torch.float32)
    ref[2 * 128 + 77:3 * 128] = 0
    ref[3 * 128:4 * 128] = 0
    assert rel(out, ref) < 1e-4
    # linear with MXFP8 forward and bf16 backward
    xl = torch.randn(4, 96, K, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    wl = (torch.randn(N, K, device="cuda") * 0.05).bfloat16().requires_grad_()
    y = mx_linear(xl, wl)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = xl.detach().float().requires_grad_(), wl.detach().float().requires_grad_()
    yr = xf @ wf.t()
    yr.backward(g.float())
    assert rel(y, yr) < 0.06 and rel(xl.grad, xf.grad) < 1e-2 and rel(wl.grad, wf.grad) < 1e-2


def test_embedding_backward_into_the_gradient_arena():
    """grad[ids[t]] += dy[t] by vector reductions into an fp32 ``main_grad``: overwrite on the first use of a step,
    accumulate afterwards (tied weights); fp32 index_add as the oracle."""
    from nanopysche_b200.ops.embedding import embedding

    torch.manual_seed(19)
    V, D = 1000, 512
    w = torch.randn(V, D, device="cuda").bfloat16().requires_grad_()
    w.main_grad = torch.full((V, D), 7.0, device="cuda")          # stale values that the first use must overwrite
    w._main_grad_dirty = False
    ids = torch.randint(0, V, (3, 700), device="cuda")
    ids[0, :50] = 5                                                # many tokens on one row
    y = embedding(ids, w)
    assert torch.equal(y, w.detach()[ids])
    g = torch.randn_like(y)
    y.backward(g)
    ref = torch.zeros(V, D, device="cuda").index_add_(0, ids.reshape(-1), g.float().reshape(-1, D))
    assert w.grad is None and w._main_grad_dirty and rel(w.main_grad, ref) < 1e-5
    embedding(ids, w).backward(g)                                  # second use in the same step accumulates
    assert rel(w.main_grad, 2 * ref) < 1e-5
    w2 = w.detach().clone().requires_grad_()                       # no arena: dense gradient through autograd
    embedding(ids, w2).backward(g)
    assert rel(w2.grad, ref) < 1e-2


@pytest.mark.parametrize("rows,D,with_res", [(300, 256, False), (4096, 2048, True), (77, 4096, True)])
def test_rmsnorm_with_fp8_output(rows, D, with_res):
    """RMSNorm (+ residual) writing e4m3 + 1x128 scales: equal, bit for bit, to quantising the plain kernel's output."""
    from fp8_flow_moe import ops as fops
    from nanopysche_b200.ops.norm import rms_norm, rms_norm_quant

    torch.manual_seed(18)
    x = (torch.randn(rows, D, device="cuda") * 2).bfloat16()
    res = torch.randn(rows, D, device="cuda").bfloat16() if with_res else None
    w = torch.rand(D, device="cuda") + 0.5
    out = rms_norm(x, w, 1e-6, res)
    y, h = out if with_res else (out, None)
    q_ref, s_ref = fops.quantize_to_fp8(y)
    got = rms_norm_quant(x, w, 1e-6, res, return_bf16=True)
    q, s = got[0], got[1]
    assert torch.equal(q.view(torch.uint8), q_ref.view(torch.uint8)) and torch.equal(s, s_ref.view_as(s))
    assert torch.equal(got[-1], y)
    if with_res:
        assert torch.equal(got[2], h)
    deq = fops.dequantize_from_fp8(q, s, dtype=torch.float32)
    assert rel(deq, y) < 0.04


@pytest.mark.parametrize("M,N,K,f32", [(300, 200, 192, False), (1024, 768, 512, True)])
def test_gemm_bias_and_residual_epilogue(M, N, K, f32):
    """Bias (per output column) and residual (same shape as the output) added in the GEMM's epilogue."""
    from nanopysche_b200.ops.gemm import gemm, linear

    torch.manual_seed(17)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = (torch.randn(N, K, device="cuda") * 0.1).bfloat16()
    bias = torch.randn(N, device="cuda")
    dt = torch.float32 if f32 else torch.bfloat16
    res = torch.randn(M, N, device="cuda").to(dt)
    ref = a.float() @ b.float().t()
    assert rel(gemm(a, b, bias=bias, out_dtype=dt), ref + bias) < 6e-3
    assert rel(gemm(a, b, residual=res, out_dtype=dt), ref + res.float()) < 6e-3
    assert rel(gemm(a, b, bias=bias, residual=res, out_dtype=dt, alpha=0.5), 0.5 * ref + bias + res.float()) < 6e-3
    x = a.view(2, M // 2, K).clone().requires_grad_()
    w = b.clone().requires_grad_()
    bb = bias.bfloat16().requires_grad_()
    y = linear(x, w, bb)
    g = torch.randn_like(y)
    y.backward(g)
    assert rel(y, ref.view(2, M // 2, N) + bb.float()) < 6e-3
    assert rel(bb.grad, g.float().sum((0, 1))) < 6e-3 and rel(w.grad, g.float().view(M, N).t() @ a.float()) < 6e-3


@pytest.mark.parametrize("recipe", ["blockwise", "mxfp8"])
def test_fp8_recipe_tag_routes_linear_to_the_fp8_gemm(recipe):
    from nanopysche_b200.ops.gemm import linear

    torch.manual_seed(16)
    x = torch.randn(3, 100, 512, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(384, 512, device="cuda") * 0.05).bfloat16().requires_grad_()
    plain = linear(x, w)
    w._fp8_recipe = recipe
    y = linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = xf @ wf.t()
    yr.backward(g.float())
    assert 1e-3 < rel(y, yr) < 0.06 and not torch.equal(y, plain)   # fp8 operands, not the bf16 GEMM
    assert rel(x.grad, xf.grad) < 1e-2 and rel(w.grad, wf.grad) < 1e-2


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,causal", [
    (1, 128, 128, 1, 1, False), (2, 512, 512, 4, 2, True), (1, 200, 200, 2, 2, True),
    (1, 128, 384, 2, 1, True), (1, 384, 256, 2, 2, False), (1, 1, 300, 4, 2, True)])
def test_flash_attention_fwd_bwd(B, Sq, Sk, Hq, Hkv, causal):
    """tcgen05 flash kernels (forward, dQ, dK/dV) against the fp32 reference of the same op."""
    from nanopysche_b200.ops import _lib
    from nanopysche_b200.ops import attention as A

    torch.manual_seed(0)
    q = torch.randn(B, Sq, Hq, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    k = torch.randn(B, Sk, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    v = torch.randn(B, Sk, Hkv, 128, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(B, Sq, Hq, 128, device="cuda", dtype=torch.bfloat16)
    assert A.flash_supported(q, k)
    o, lse = A.flash_fwd(q.detach(), k.detach(), v.detach(), causal=causal, q_off=(Sk - Sq) if causal else 0)
    A.attention(q, k, v, causal=causal).backward(g)     # the public op takes the same kernels
    torch.cuda.synchronize()
    _lib.check_status("flash")
    qf, kf, vf = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ro, rl = A.attention_ref(qf, kf, vf, causal=causal)
    ro.backward(g.float())
    assert (o.float() - ro).abs().max().item() < 3e-2
    assert (lse - rl).abs().max().item() < 1e-3
    for got, ref in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        assert ((got.float() - ref).abs().max() / ref.abs().max()).item() < 2e-2


def test_flash_attention_strided_qkv_views():
    """q / k / v as slices of one fused projection output (no copies) give the same result."""
    from nanopysche_b200.ops import attention as A

    torch.manual_seed(1)
    B, S, Hq, Hkv = 2, 256, 4, 2
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[..., : Hq * 128].unflatten(-1, (Hq, 128))
    k = qkv[..., Hq * 128:(Hq + Hkv) * 128].unflatten(-1, (Hkv, 128))
    v = qkv[..., (Hq + Hkv) * 128:].unflatten(-1, (Hkv, 128))
    o, _ = A.flash_fwd(q, k, v, causal=True)
    o2, _ = A.flash_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal=True)
    assert torch.equal(o, o2)


def test_qkv_layernorm_rope_fused_matches_unfused():
    """Fused split + q/k LayerNorm + RoPE (forward and backward) against the unfused module math in fp32."""
    from nanopysche_b200.models.attention import Attention
    from nanopysche_b200.ops import rope as rope_ops

    torch.manual_seed(0)
    B, S, hq, hkv, hd = 2, 96, 4, 2, 128
    att = Attention(d_model=hq * hd, n_heads=hq, n_kv_heads=hkv, qk_norm=True, device="cuda")
    with torch.no_grad():
        for ln in (att.q_norm, att.k_norm):
            ln.weight.normal_(1.0, 0.2)
            ln.bias.normal_(0.0, 0.2)
    cos, sin = att.rope.half_tables(S + 5, torch.device("cuda"))
    qkv = torch.randn(B, S, (hq + 2 * hkv) * hd, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    assert rope_ops.qkv_norm_rope_supported(qkv, cos, hq, hkv, hd)
    q, k, v = rope_ops.qkv_norm_rope(qkv, att.q_norm, att.k_norm, cos, sin, hq, hkv, 5, None)
    gq, gk, gv = torch.randn_like(q), torch.randn_like(k), torch.randn_like(v)
    torch.autograd.backward([q, k, v], [gq, gk, gv])
    got = [qkv.grad.clone(), att.q_norm.weight.grad.clone(), att.q_norm.bias.grad.clone(),
           att.k_norm.weight.grad.clone(), att.k_norm.bias.grad.clone()]
    qkv.grad = None
    for ln in (att.q_norm, att.k_norm):
        ln.weight.grad = ln.bias.grad = None
    # reference: slice, LayerNorm in fp32, rotate with the reference rotation, all in fp32
    x = qkv.detach().float().requires_grad_()
    q0 = x[..., : hq * hd].unflatten(-1, (hq, hd))
    k0 = x[..., hq * hd:(hq + hkv) * hd].unflatten(-1, (hkv, hd))
    v0 = x[..., (hq + hkv) * hd:].unflatten(-1, (hkv, hd))
    qr = rope_ops.apply_rope_ref(att.q_norm(q0), cos, sin, 5, None)
    kr = rope_ops.apply_rope_ref(att.k_norm(k0), cos, sin, 5, None)
    torch.autograd.backward([qr, kr, v0], [gq.float(), gk.float(), gv.float()])
    assert (q.float() - qr).abs().max().item() < 5e-2 and (k.float() - kr).abs().max().item() < 5e-2
    assert torch.equal(v, v0.detach().to(v.dtype))
    ref = [x.grad, att.q_norm.weight.grad, att.q_norm.bias.grad, att.k_norm.weight.grad, att.k_norm.bias.grad]
    for a, b in zip(got, ref):
        assert ((a.float() - b.float()).norm() / b.float().norm()).item() < 1.5e-2


def test_flow_moe_power_of_two_block_quantisers_and_gemm():
    """FP8-Flow-MoE blocks on the block-scaled tensor-core path: the 1x128 activation quantiser (plain and fused with
    SwiGLU), the 128x128 weight quantiser (plain, stacked output, per-expert transpose) and the dequantiser are
    bit-exact against their PyTorch statements; the GEMM on their outputs matches the fp32 product of the dequantised
    operands; and the end-to-end error against the unquantised product is at the e4m3 level."""
    from nanopysche_b200.ops import gemm_mxfp8 as mx

    torch.manual_seed(0)
    rows, K, H, E = 384, 512, 256, 2
    x = (torch.randn(rows, K, device="cuda") * torch.rand(rows, 1, device="cuda") * 4).bfloat16()
    q, sf = mx.flow_quantize_act(x)
    qr, sfr = mx.flow_quantize_act_ref(x)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8)) and torch.equal(sf, sfr)
    assert torch.equal(mx.mx_dequantize_bf16(q, sf), mx.mx_dequantize(qr, sfr).bfloat16())
    gu = torch.randn(200, 2 * H, device="cuda").bfloat16()
    hq, hs = mx.flow_quantize_act(gu, swiglu=True)
    hqr, hsr = mx.flow_quantize_act_ref(gu, swiglu=True)
    d, dr = mx.mx_dequantize(hq, hs), mx.mx_dequantize(hqr, hsr)
    assert rel(d, dr) < 2e-2   # silu goes through __expf on the device: values may land in a neighbouring e4m3 code
    w = (torch.randn(E * H, K, device="cuda") * 0.05).bfloat16()
    for tr in (False, True):
        wq, ws = mx.flow_quantize_weight(w, E, tr)
        wqr, wsr = mx.flow_quantize_weight_ref(w, E, tr)
        assert torch.equal(wq.view(torch.uint8), wqr.view(torch.uint8)) and torch.equal(ws, wsr), tr
    # stacked output: [w_a; w_b] per expert in one matrix
    wb = (torch.randn(E * H, K, device="cuda") * 0.05).bfloat16()
    q2 = torch.empty((E * 2 * H, K), device="cuda", dtype=torch.float8_e4m3fn)
    s2 = torch.zeros(mx.sf_bytes(E * 2 * H, K), device="cuda", dtype=torch.uint8)
    mx.flow_quantize_weight(w, E, out=(q2, s2), out_rows=2 * H, out_row0=0)
    mx.flow_quantize_weight(wb, E, out=(q2, s2), out_rows=2 * H, out_row0=H)
    stacked = torch.cat([w.view(E, H, K), wb.view(E, H, K)], dim=1).reshape(E * 2 * H, K)
    q2r, s2r = mx.flow_quantize_weight_ref(stacked, E)
    assert torch.equal(q2.view(torch.uint8), q2r.view(torch.uint8)) and torch.equal(s2, s2r)
    # grouped GEMM: 3 row blocks over 2 experts, N = 2H per expert
    grp = torch.tensor([0, 1, 1], device="cuda", dtype=torch.int32)
    got = mx.gemm_mxfp8(q, sf, q2, s2, mblk_group=grp, rows_per_group=2 * H, out_dtype=torch.float32)
    ref = mx.gemm_mxfp8_ref(q, sf, q2, s2, grp, 2 * H, torch.float32)
    assert rel(got, ref) < 1e-4
    exact = torch.cat([x[i * 128:(i + 1) * 128].float() @ stacked.view(E, 2 * H, K)[g].float().t()
                       for i, g in enumerate(grp.tolist())])
    assert rel(got, exact) < 0.06


def test_attention_head_dim_64_runs_on_the_flash_kernels_padded():
    """head_dim 64 (the 125m / 350m / 1b presets): ``ops.attention.attention`` zero-pads the head dimension to 128
    and runs the tcgen05 kernels; output and gradients match fp32 SDPA."""
    from nanopysche_b200.ops import _lib
    from nanopysche_b200.ops.attention import attention

    torch.manual_seed(0)
    B, S, Hq, Hkv, hd = 2, 384, 4, 2, 64
    q = torch.randn(B, S, Hq, hd, device="cuda").bfloat16().requires_grad_(True)
    k = torch.randn(B, S, Hkv, hd, device="cuda").bfloat16().requires_grad_(True)
    v = torch.randn(B, S, Hkv, hd, device="cuda").bfloat16().requires_grad_(True)
    l0 = _lib.LAUNCHES
    o = attention(q, k, v, causal=True)
    assert _lib.LAUNCHES > l0 and o.shape == (B, S, Hq, hd)
    g = torch.randn_like(o)
    o.backward(g)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    of = torch.nn.functional.scaled_dot_product_attention(qf.transpose(1, 2), kf.transpose(1, 2), vf.transpose(1, 2),
                                                          is_causal=True, enable_gqa=True).transpose(1, 2)
    of.backward(g.float())
    assert rel(o, of) < 2e-2
    for a, b in ((q, qf), (k, kf), (v, vf)):
        assert rel(a.grad, b.grad) < 3e-2


@pytest.mark.parametrize("M,N,K", [(512, 512, 128), (600, 520, 200), (4096, 2048, 2048), (1000, 32000, 256)])
def test_gemm_256_row_tiles_all_layouts(M, N, K):
    """The 256 x 256 tile form (two 128-row halves sharing every B tile, single-buffered accumulators), forced on,
    against fp32 matmul: forward, dgrad and wgrad operand layouts, fp32 accumulate, ragged edges."""
    from nanopysche_b200.ops.gemm import gemm

    torch.manual_seed(0)
    a = torch.randn(M, K, device="cuda").bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    ref = a.float() @ b.float().t()
    assert rel(gemm(a, b, bn=256, mt=2), ref) < 1e-2
    assert rel(gemm(a, b.t().contiguous(), b_mn=True, bn=256, mt=2), ref) < 1e-2                    # dgrad layout
    at, bt = a.t().contiguous(), b.t().contiguous()
    out = torch.full((M, N), 0.5, device="cuda")
    gemm(at, bt, a_mn=True, b_mn=True, out=out, accumulate=True, bn=256, mt=2)                     # wgrad layout, +=
    assert rel(out, ref + 0.5) < 1e-2
    assert rel(gemm(a, b, bn=256, mt=2), gemm(a, b, bn=256, mt=1)) < 1e-5                          # same numbers as 128-row tiles
