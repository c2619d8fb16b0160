"""Kernel micro-benchmarks: ``python -m benchmarks.microbench <case> [options]`` (from the repository root).

Each case times one in-tree kernel with CUDA events after warm-up, flushing L2 between iterations
(a 512 MB write), and prints one JSON line with the achieved rate and its fraction of the measured
roofline (``MEASURED_PEAKS.json`` at the repository root when present, else 6.65 TB/s and
1.59 PFLOP/s). The same command lines are what the ``ncu`` captures under ``profiles/`` run.

Cases: gemm (fwd / dgrad / wgrad layouts, optional cuBLAS comparison), swiglu (fused GEMM + SwiGLU),
rmsnorm, adamw, xent, moe (one fused MoE layer forward + backward), attention (flash forward / backward), mxfp8,
flow (the FP8-Flow-MoE grouped expert GEMMs against the bf16 grouped GEMM at the same shapes).
"""
from __future__ import annotations

import argparse
import json
import os
from pathlib import Path

import torch


def peaks():
    p = Path(__file__).resolve().parents[1] / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return d.get("hbm_gbs", 6650.0), d.get("bf16_tflops", 1590.0), "measured"
    return 6650.0, 1590.0, "fallback"


def timeit(fn, iters: int, warmup: int = 3, flush: bool = True):
    scratch = torch.empty(512 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush:
            scratch.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    times.sort()
    return times[len(times) // 2], times[0]


def case_gemm(a):
    from nanopysche_b200.ops.gemm import gemm

    M, N, K = a.m, a.n, a.k
    dev = "cuda"
    if a.layout == "fwd":
        A, B = torch.randn(M, K, device=dev).bfloat16(), torch.randn(N, K, device=dev).bfloat16()
        kw, ref = {}, (lambda: torch.matmul(A, B.t()))
    elif a.layout == "dgrad":
        A, B = torch.randn(M, K, device=dev).bfloat16(), torch.randn(K, N, device=dev).bfloat16()
        kw, ref = dict(b_mn=True), (lambda: torch.matmul(A, B))
    else:
        A, B = torch.randn(K, M, device=dev).bfloat16(), torch.randn(K, N, device=dev).bfloat16()
        kw, ref = dict(a_mn=True, b_mn=True), (lambda: torch.matmul(A.t(), B))
    out = torch.empty(M, N, device=dev, dtype=torch.float32 if a.f32 else torch.bfloat16)
    med, best = timeit(lambda: gemm(A, B, out=out, bn=a.bn, **kw), a.iters)
    flops = 2.0 * M * N * K
    res = {"case": "gemm", "layout": a.layout, "M": M, "N": N, "K": K, "ms": med, "ms_best": best,
           "tflops": flops / med / 1e9}
    if a.cublas:
        m2, _ = timeit(ref, a.iters)
        res["cublas_ms"], res["cublas_tflops"] = m2, flops / m2 / 1e9
    return res, flops, None


def case_swiglu(a):
    from nanopysche_b200.ops.gemm import gemm_swiglu

    x = torch.randn(a.m, a.k, device="cuda").bfloat16()
    w1 = torch.randn(a.n, a.k, device="cuda").bfloat16()
    w3 = torch.randn(a.n, a.k, device="cuda").bfloat16()
    med, best = timeit(lambda: gemm_swiglu(x, w1, w3, save_gu=not a.no_gu), a.iters)
    flops = 4.0 * a.m * a.n * a.k
    return {"case": "swiglu", "M": a.m, "N": a.n, "K": a.k, "ms": med, "tflops": flops / med / 1e9}, flops, None


def case_rmsnorm(a):
    from nanopysche_b200.ops.norm import rms_norm

    x = torch.randn(a.m, a.n, device="cuda").bfloat16()
    r = torch.randn(a.m, a.n, device="cuda").bfloat16()
    w = torch.ones(a.n, device="cuda")
    med, best = timeit(lambda: rms_norm(x, w, 1e-6, r), a.iters)
    nbytes = a.m * a.n * 2 * 4  # read x, res; write y, h
    return {"case": "rmsnorm", "rows": a.m, "cols": a.n, "ms": med, "gbs": nbytes / med / 1e6}, None, nbytes


def case_adamw(a):
    from nanopysche_b200.ops import _lib

    n = a.m * a.n
    p, g = torch.randn(n, device="cuda"), torch.randn(n, device="cuda")
    m, v = torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    w16 = torch.empty(n, device="cuda", dtype=torch.bfloat16)
    med, best = timeit(lambda: _lib.call("adamw", p, g, m, v, w16, _lib.LL(n), 1e-3, 0.9, 0.95, 1e-8, 0.1, 1, None,
                                         None), a.iters)
    nbytes = n * 30
    return {"case": "adamw", "n": n, "ms": med, "gbs": nbytes / med / 1e6}, None, nbytes


def case_xent(a):
    from nanopysche_b200.ops.xent import cross_entropy

    logits = torch.randn(a.m, a.n, device="cuda").bfloat16().requires_grad_(True)
    labels = torch.randint(0, a.n, (a.m,), device="cuda")

    def run():
        cross_entropy(logits, labels).backward()
        logits.grad = None

    med, best = timeit(run, a.iters)
    nbytes = a.m * a.n * 2 * 4  # fwd reads twice, bwd reads once and writes once
    return {"case": "xent", "rows": a.m, "V": a.n, "ms": med, "gbs": nbytes / med / 1e6}, None, nbytes


def case_moe(a):
    from nanopysche_b200.models.moe import MoEBase
    from nanopysche_b200.ops.moe import build_runtime

    T, D, H, E, K = a.m, a.k, a.n, a.experts, a.topk
    moe = MoEBase(d_model=D, hidden_size=H, num_experts=E, top_k=K, capacity_factor=a.capacity, dtype=torch.bfloat16,
                  device="cuda", init_std=0.02)
    for w in (moe.w1, moe.w2, moe.w3):
        w.main_grad = torch.zeros(w.shape, device="cuda")
    build_runtime([moe], tokens=T, device=torch.device("cuda"))
    x = torch.randn(1, T, D, device="cuda").bfloat16().requires_grad_(True)
    gy = torch.randn(1, T, D, device="cuda").bfloat16()

    def run():
        for w in (moe.w1, moe.w2, moe.w3):
            w._main_grad_dirty = False
        moe(x).backward(gy)
        x.grad = None

    med, best = timeit(run, a.iters)

    def fwd():
        with torch.no_grad():
            moe(x)

    fmed, _ = timeit(fwd, a.iters)
    kept = T * K if a.capacity is None else min(T * K, E * int(a.capacity * T / E))
    flops = 3.0 * kept * 6.0 * D * H
    return {"case": "moe", "T": T, "D": D, "H": H, "E": E, "K": K, "capacity": a.capacity, "ms": med,
            "fwd_ms": fmed, "fwd_tokens_per_s": T / fmed * 1e3,
            "tflops_upper_bound_rows": flops / med / 1e9}, None, None


def case_attention(a):
    """Flash attention forward and backward (``--batch --seq --heads --kv-heads``, head_dim 128, causal unless
    ``--full``); ``--sdpa`` also times PyTorch SDPA on the same tensors. FLOPs: 4 B H S^2 hd (x 2.5 for backward),
    halved under causal masking."""
    from nanopysche_b200.ops import attention as A

    B, S, Hq, Hkv = a.batch, a.seq, a.heads, a.kv_heads
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * 128, device="cuda", dtype=torch.bfloat16)
    q = qkv[..., : Hq * 128].unflatten(-1, (Hq, 128))
    k = qkv[..., Hq * 128:(Hq + Hkv) * 128].unflatten(-1, (Hkv, 128))
    v = qkv[..., (Hq + Hkv) * 128:].unflatten(-1, (Hkv, 128))
    g = torch.randn(B, S, Hq, 128, device="cuda", dtype=torch.bfloat16)
    causal = not a.full
    o, lse = A.flash_fwd(q, k, v, causal=causal)
    fwd, _ = timeit(lambda: A.flash_fwd(q, k, v, causal=causal), a.iters)
    bwd, _ = timeit(lambda: A.flash_bwd(q, k, v, o, g, lse, causal=causal), a.iters)
    fl = 4.0 * B * Hq * S * S * 128 * (0.5 if causal else 1.0)
    res = {"case": "attention", "B": B, "S": S, "Hq": Hq, "Hkv": Hkv, "causal": causal, "fwd_ms": fwd, "bwd_ms": bwd,
           "ms": fwd, "tflops": fl / fwd / 1e9, "bwd_tflops": 2.5 * fl / bwd / 1e9}
    if a.sdpa:
        qs, ks, vs = [t.detach().clone().requires_grad_() for t in (q, k, v)]
        os_ = torch.nn.functional.scaled_dot_product_attention(
            qs.transpose(1, 2), ks.transpose(1, 2), vs.transpose(1, 2), is_causal=causal, enable_gqa=Hq != Hkv)
        f2, _ = timeit(lambda: torch.nn.functional.scaled_dot_product_attention(
            qs.transpose(1, 2), ks.transpose(1, 2), vs.transpose(1, 2), is_causal=causal, enable_gqa=Hq != Hkv), a.iters)
        b2, _ = timeit(lambda: torch.autograd.grad(os_, (qs, ks, vs), g.transpose(1, 2), retain_graph=True), a.iters)
        res["sdpa_fwd_ms"], res["sdpa_bwd_ms"] = f2, b2
    return res, fl, None


def case_mxfp8(a):
    """MXFP8 GEMM (operands quantised beforehand), the quantiser alone, and the block-scaled 1x128 kernel."""
    from nanopysche_b200.ops.gemm_mxfp8 import gemm_mxfp8, mx_quantize

    M, N, K = a.m, a.n, a.k
    A, B = torch.randn(M, K, device="cuda").bfloat16(), torch.randn(N, K, device="cuda").bfloat16()
    aq, sa = mx_quantize(A)
    bq, sb = mx_quantize(B)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    med, best = timeit(lambda: gemm_mxfp8(aq, sa, bq, sb, out=out), a.iters)
    qmed, _ = timeit(lambda: mx_quantize(A), a.iters)
    flops = 2.0 * M * N * K
    res = {"case": "mxfp8", "M": M, "N": N, "K": K, "ms": med, "ms_best": best, "tflops": flops / med / 1e9,
           "quant_ms": qmed, "quant_gbs": M * K * 3.03 / qmed / 1e6}
    if a.cublas:
        from fp8_flow_moe import ops as fops

        from nanopysche_b200.ops.gemm_fp8 import gemm_fp8_block

        xq, xs = fops.quantize_to_fp8(A)
        wq, ws = fops.quantize_weight_blockwise(B)
        m2, _ = timeit(lambda: gemm_fp8_block(xq, xs, wq, ws, out=out), a.iters)
        res["block128_ms"], res["block128_tflops"] = m2, flops / m2 / 1e9
        m3, _ = timeit(lambda: torch.matmul(A, B.t()), a.iters)
        res["cublas_bf16_ms"], res["cublas_bf16_tflops"] = m3, flops / m3 / 1e9
    return res, flops, None


def case_flow(a):
    """Grouped expert GEMMs of one MoE layer at ``--m`` rows per expert, ``--experts`` local experts, d_model
    ``--k``, expert hidden ``--n``: gate|up (``[rows, 2H] = x @ [w1; w3]^T``) and down (``[rows, D] = h @ w2``) on
    the block-scaled e4m3 path (1x128 / 128x128 power-of-two scales) and on the bf16 tcgen05 path, plus the
    quantisers the fp8 path adds (SwiGLU + re-quantise per forward, weights once per optimizer step)."""
    from nanopysche_b200.ops import _lib
    from nanopysche_b200.ops import gemm_mxfp8 as mx
    import ctypes as C

    E, R, D, H = a.experts, a.m, a.k, a.n
    rows = E * R
    dev = "cuda"
    x = torch.randn(rows, D, device=dev).bfloat16()
    w1, w3, w2 = (torch.randn(E * H, D, device=dev).bfloat16() * 0.02 for _ in range(3))
    grp = torch.arange(E, device=dev, dtype=torch.int32).repeat_interleave(R // 128)
    mrows = torch.full((rows // 128,), 128, device=dev, dtype=torch.int32)
    xq, xs = mx.flow_quantize_act(x)
    w13q = torch.empty((E * 2 * H, D), device=dev, dtype=torch.float8_e4m3fn)
    s13 = torch.zeros(mx.sf_bytes(E * 2 * H, D), device=dev, dtype=torch.uint8)
    mx.flow_quantize_weight(w1, E, out=(w13q, s13), out_rows=2 * H, out_row0=0)
    mx.flow_quantize_weight(w3, E, out=(w13q, s13), out_rows=2 * H, out_row0=H)
    w2q, s2 = mx.flow_quantize_weight(w2, E, transpose=True)
    gu = torch.empty(rows, 2 * H, device=dev, dtype=torch.bfloat16)
    y = torch.empty(rows, D, device=dev, dtype=torch.bfloat16)
    t_gu, _ = timeit(lambda: mx.gemm_mxfp8(xq, xs, w13q, s13, out=gu, mblk_group=grp, mblk_rows=mrows,
                                           rows_per_group=2 * H), a.iters)
    hq, hs = mx.flow_quantize_act(gu, swiglu=True)
    t_q, _ = timeit(lambda: mx.flow_quantize_act(gu, swiglu=True, out=(hq, hs)), a.iters)
    t_dn, _ = timeit(lambda: mx.gemm_mxfp8(hq, hs, w2q, s2, out=y, mblk_group=grp, mblk_rows=mrows, rows_per_group=D),
                     a.iters)
    t_wq, _ = timeit(lambda: (mx.flow_quantize_weight(w1, E, out=(w13q, s13), out_rows=2 * H, out_row0=0),
                              mx.flow_quantize_weight(w3, E, out=(w13q, s13), out_rows=2 * H, out_row0=H),
                              mx.flow_quantize_weight(w2, E, transpose=True, out=(w2q, s2))), a.iters)

    def bf16_grouped(A, B, N, K, b_mn, out, B2=None, C2=None):
        g = _lib.GemmArgs()
        g.A, g.B, g.C = A.data_ptr(), B.data_ptr(), out.data_ptr()
        g.lda, g.ldb, g.ldc = A.stride(0), B.stride(0), out.stride(0)
        g.a_rows, g.b_rows, g.M, g.N, g.K = A.shape[0], B.shape[0], rows, N, K
        g.b_mn, g.mode, g.alpha = int(b_mn), 1, 1.0
        g.mblk_group, g.mblk_rows, g.group_stride_b = grp.data_ptr(), mrows.data_ptr(), H
        if B2 is not None:
            g.B2, g.epilogue, g.C2, g.ldc2 = B2.data_ptr(), 1, C2.data_ptr(), C2.stride(0)
        _lib.check(_lib.lib().np_gemm_bf16(C.byref(g), C.c_void_p(_lib.stream())), "grouped_gemm")

    h = torch.empty(rows, H, device=dev, dtype=torch.bfloat16)
    b_gu, _ = timeit(lambda: bf16_grouped(x, w1, H, D, False, h, B2=w3, C2=gu), a.iters)
    b_dn, _ = timeit(lambda: bf16_grouped(h, w2, D, H, True, y), a.iters)
    f_gu, f_dn = 2.0 * rows * 2 * H * D, 2.0 * rows * D * H
    res = {"case": "flow", "rows_per_expert": R, "experts": E, "D": D, "H": H,
           "fp8_gate_up_ms": t_gu, "fp8_gate_up_tflops": f_gu / t_gu / 1e9,
           "fp8_down_ms": t_dn, "fp8_down_tflops": f_dn / t_dn / 1e9,
           "swiglu_quant_ms": t_q, "weight_quant_ms_per_step": t_wq,
           "bf16_gate_up_swiglu_ms": b_gu, "bf16_gate_up_tflops": f_gu / b_gu / 1e9,
           "bf16_down_ms": b_dn, "bf16_down_tflops": f_dn / b_dn / 1e9,
           "gemm_speedup_gate_up": b_gu / t_gu, "gemm_speedup_down": b_dn / t_dn,
           "forward_speedup_with_quant": (b_gu + b_dn) / (t_gu + t_q + t_dn),
           "ms": t_gu + t_dn, "tflops": (f_gu + f_dn) / (t_gu + t_dn) / 1e9}
    return res, f_gu + f_dn, None


CASES = {"flow": case_flow, "mxfp8": case_mxfp8, "attention": case_attention, "gemm": case_gemm, "swiglu": case_swiglu, "rmsnorm": case_rmsnorm, "adamw": case_adamw, "xent": case_xent,
         "moe": case_moe}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--m", type=int, default=4096)
    ap.add_argument("--n", type=int, default=5632)
    ap.add_argument("--k", type=int, default=2048)
    ap.add_argument("--bn", type=int, default=0)
    ap.add_argument("--layout", choices=["fwd", "dgrad", "wgrad"], default="fwd")
    ap.add_argument("--f32", action="store_true", help="fp32 output")
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul")
    ap.add_argument("--no-gu", action="store_true")
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--topk", type=int, default=2)
    ap.add_argument("--capacity", type=float, default=None)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--heads", type=int, default=16)
    ap.add_argument("--kv-heads", type=int, default=8)
    ap.add_argument("--full", action="store_true", help="attention without the causal mask")
    ap.add_argument("--sdpa", action="store_true", help="also time PyTorch SDPA")
    a = ap.parse_args(argv)
    hbm, tf, src = peaks()
    res, flops, nbytes = CASES[a.case](a)
    if flops:
        res["frac_of_" + src + "_bf16_peak"] = res.get("tflops", 0.0) / tf
    if nbytes:
        res["frac_of_" + src + "_hbm"] = res["gbs"] / hbm
    from nanopysche_b200.ops import _lib

    res["status"] = list(_lib.status())
    print(json.dumps(res))


if __name__ == "__main__":
    main()
