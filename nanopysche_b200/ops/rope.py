"""Rotary position embedding: table generation and the half-split rotation, forward and backward.

Reference math: model/rope.py:62-106 (inv_freq, optional piecewise scaling, cos/sin of
``outer(pos, inv_freq)``) and :139-170 (``x*cos + rotate_half(x)*sin``, halves split at ``rot/2``).
The sm_100a kernel (csrc/elementwise.cu ``rope_kernel``) rotates a strided ``[T, H, hd]`` view, so it
runs directly on the q and k slices of a fused QKV GEMM output; the backward pass is the same kernel
with the sine negated. ``yarn`` adds the NTK-by-parts ramp and attention scale that the reference's
"YaRN" lacks.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib

SCALING_IDS = {None: 0, "none": 0, "piecewise": 1, "yarn": 2}


def yarn_mscale(factor: float) -> float:
    return 1.0 if factor <= 1.0 else 0.1 * math.log(factor) + 1.0


def rope_tables_ref(seq_len: int, rot: int, base: float = 10000.0, scaling: str | None = None,
                    factor: float = 1.0, orig_len: float = 8192.0, low_f: float = 1.0, high_f: float = 4.0,
                    device="cpu"):
    """(cos, sin), each fp32 ``[seq_len, rot/2]``."""
    half = rot // 2
    idx = torch.arange(half, dtype=torch.float32, device=device)
    inv = base ** (-2.0 * idx / rot)
    ms = 1.0
    if scaling == "piecewise" and factor > 1.0:
        wavelen = 2 * math.pi / inv
        inv = torch.where(wavelen < orig_len / high_f, inv,
                          torch.where(wavelen > orig_len / low_f, inv / factor, inv))
    elif scaling == "yarn" and factor > 1.0:
        d_lo = rot * math.log(orig_len / (high_f * 2 * math.pi)) / (2 * math.log(base))
        d_hi = rot * math.log(orig_len / (low_f * 2 * math.pi)) / (2 * math.log(base))
        lo, hi = max(math.floor(d_lo), 0), min(math.ceil(d_hi), half - 1)
        ramp = ((idx - lo) / max(hi - lo, 1e-3)).clamp(0, 1)
        extrap = 1.0 - ramp
        inv = (inv / factor) * (1 - extrap) + inv * extrap
        ms = yarn_mscale(factor)
    ang = torch.outer(torch.arange(seq_len, dtype=torch.float32, device=device), inv)
    return ang.cos() * ms, ang.sin() * ms


def rope_tables(seq_len, rot, base=10000.0, scaling=None, factor=1.0, orig_len=8192.0, low_f=1.0, high_f=4.0,
                device="cpu"):
    dev = torch.device(device)
    if dev.type != "cuda":
        return rope_tables_ref(seq_len, rot, base, scaling, factor, orig_len, low_f, high_f, device)
    cos = torch.empty((seq_len, rot // 2), device=dev, dtype=torch.float32)
    sin = torch.empty_like(cos)
    sid = SCALING_IDS[scaling] if factor > 1.0 else 0
    if sid == 2:  # yarn: low_f/high_f are beta_slow/beta_fast
        ms = yarn_mscale(factor)
    else:
        ms = 1.0
    _lib.call("rope_table", cos, sin, seq_len, rot, float(base), sid, float(factor), float(orig_len),
              float(low_f), float(high_f), float(ms))
    return cos, sin


def apply_rope_ref(x, cos, sin, pos_offset: int = 0, pos_ids=None, sign: float = 1.0):
    """x: [B, S, H, hd]; cos/sin: [max_pos, rot/2]."""
    B, S, H, hd = x.shape
    half = cos.shape[1]
    rot = 2 * half
    if pos_ids is None:
        pos = torch.arange(S, device=x.device) + pos_offset
        c, s = cos[pos][None, :, None, :], sin[pos][None, :, None, :]
    else:
        p = pos_ids.reshape(B, S).long()
        c, s = cos[p][:, :, None, :], sin[p][:, :, None, :]
    s = s * sign
    xf = x.float()
    x1, x2, rest = xf[..., :half], xf[..., half:rot], xf[..., rot:]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s, rest], dim=-1)
    return out.to(x.dtype)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, pos_offset, pos_ids, inplace):
        B, S, H, hd = x.shape
        assert x.stride(3) == 1 and x.stride(2) == hd and x.stride(0) == S * x.stride(1)
        out = x if inplace else torch.empty((B, S, H, hd), device=x.device, dtype=x.dtype)
        _lib.call("rope", x, out, cos, sin, pos_ids, _lib.LL(B * S), S, int(pos_offset), H, hd, 2 * cos.shape[1],
                  _lib.LL(x.stride(1)), _lib.LL(out.stride(1)), 1.0)
        ctx.save_for_backward(cos, sin, pos_ids if pos_ids is not None else cos.new_empty(0))
        ctx.meta = (pos_offset, pos_ids is not None)
        if inplace:
            ctx.mark_dirty(x)
        return out

    @staticmethod
    def backward(ctx, dy):
        cos, sin, pos_ids = ctx.saved_tensors
        pos_offset, has_ids = ctx.meta
        B, S, H, hd = dy.shape
        if not (dy.stride(3) == 1 and dy.stride(2) == hd and dy.stride(0) == S * dy.stride(1)):
            dy = dy.contiguous()
        dx = torch.empty((B, S, H, hd), device=dy.device, dtype=dy.dtype)
        _lib.call("rope", dy, dx, cos, sin, pos_ids if has_ids else None, _lib.LL(B * S), S, int(pos_offset), H, hd,
                  2 * cos.shape[1], _lib.LL(dy.stride(1)), _lib.LL(dx.stride(1)), -1.0)
        return dx, None, None, None, None, None


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos_offset: int = 0,
               pos_ids: torch.Tensor | None = None) -> torch.Tensor:
    """Rotate ``x [B, S, H, hd]`` (a possibly strided view with contiguous heads) by its positions."""
    B, S, H, hd = x.shape
    ok = (_lib.on(x) and x.dtype == torch.bfloat16 and hd % 8 == 0 and (2 * cos.shape[1]) % 16 == 0 and
          x.stride(3) == 1 and x.stride(2) == hd and x.stride(1) % 8 == 0 and x.stride(0) == S * x.stride(1) and
          cos.dtype == torch.float32)
    if ok:
        if pos_ids is not None:
            pos_ids = pos_ids.reshape(-1).to(torch.int32)
        return _Rope.apply(x, cos, sin, pos_offset, pos_ids, False)
    return apply_rope_ref(x, cos, sin, pos_offset, pos_ids)


class _QKVRope(torch.autograd.Function):
    """Split the fused QKV GEMM output into q / k / v and rotate q and k, one kernel each way."""

    @staticmethod
    def forward(ctx, qkv, cos, sin, hq, hkv, hd, pos_offset, pos_ids):
        B, S, W = qkv.shape
        H = hq + 2 * hkv
        out = torch.empty((B, S, H, hd), device=qkv.device, dtype=qkv.dtype)
        rs = qkv.stride(1)
        base = qkv.data_ptr()
        es = qkv.element_size()
        _lib.check(_lib.lib().np_qkv_rope(
            C.c_void_p(base), C.c_longlong(rs), C.c_longlong(hd), hq,
            C.c_void_p(base + hq * hd * es), C.c_longlong(rs), C.c_longlong(hd), hkv,
            C.c_void_p(base + (hq + hkv) * hd * es), C.c_longlong(rs), C.c_longlong(hd), hkv,
            C.c_void_p(out.data_ptr()), C.c_void_p(cos.data_ptr()), C.c_void_p(sin.data_ptr()),
            C.c_void_p(pos_ids.data_ptr() if pos_ids is not None else 0), C.c_longlong(B * S), S, int(pos_offset), hd,
            2 * cos.shape[1], hq + hkv, C.c_float(1.0), C.c_void_p(_lib.stream())), "qkv_rope")
        ctx.save_for_backward(cos, sin, pos_ids if pos_ids is not None else cos.new_empty(0))
        ctx.meta = (hq, hkv, hd, pos_offset, pos_ids is not None, qkv.shape)
        return out[:, :, :hq], out[:, :, hq:hq + hkv], out[:, :, hq + hkv:]

    @staticmethod
    def backward(ctx, dq, dk, dv):
        cos, sin, pos_ids = ctx.saved_tensors
        hq, hkv, hd, pos_offset, has_ids, shape = ctx.meta
        B, S, W = shape
        fixed = []
        for g, h in ((dq, hq), (dk, hkv), (dv, hkv)):
            if g is None:
                g = torch.zeros((B, S, h, hd), device=cos.device, dtype=torch.bfloat16)
            if g.stride(3) != 1 or g.stride(0) != S * g.stride(1) or g.stride(1) % 8 or g.stride(2) % 8:
                g = g.contiguous()
            fixed.append(g)
        dq, dk, dv = fixed
        out = torch.empty((B, S, W), device=dq.device, dtype=dq.dtype)
        _lib.check(_lib.lib().np_qkv_rope(
            C.c_void_p(dq.data_ptr()), C.c_longlong(dq.stride(1)), C.c_longlong(dq.stride(2)), hq,
            C.c_void_p(dk.data_ptr()), C.c_longlong(dk.stride(1)), C.c_longlong(dk.stride(2)), hkv,
            C.c_void_p(dv.data_ptr()), C.c_longlong(dv.stride(1)), C.c_longlong(dv.stride(2)), hkv,
            C.c_void_p(out.data_ptr()), C.c_void_p(cos.data_ptr()), C.c_void_p(sin.data_ptr()),
            C.c_void_p(pos_ids.data_ptr() if has_ids else 0), C.c_longlong(B * S), S, int(pos_offset), hd,
            2 * cos.shape[1], hq + hkv, C.c_float(-1.0), C.c_void_p(_lib.stream())), "qkv_rope_bwd")
        return out, None, None, None, None, None, None, None


class _QKVNormRope(torch.autograd.Function):
    """Split the fused QKV output, apply the per-head LayerNorms of q and k and rotate, one kernel each way."""

    @staticmethod
    def forward(ctx, qkv, gq, bq, gk, bk, eps, cos, sin, hq, hkv, pos_offset, pos_ids):
        B, S, W = qkv.shape
        hd, H = 128, hq + 2 * hkv
        out = torch.empty((B, S, H, hd), device=qkv.device, dtype=qkv.dtype)
        stats = torch.empty((B * S, hq + hkv, 2), device=qkv.device, dtype=torch.float32)
        f = [t.detach().float().contiguous() for t in (gq, bq, gk, bk)]
        pid = C.c_void_p(pos_ids.data_ptr() if pos_ids is not None else 0)
        _lib.check(_lib.lib().np_qkv_norm_rope_fwd(
            C.c_void_p(qkv.data_ptr()), C.c_longlong(qkv.stride(1)), hq, hkv, *[C.c_void_p(t.data_ptr()) for t in f],
            C.c_float(eps), C.c_void_p(out.data_ptr()), C.c_void_p(stats.data_ptr()), C.c_void_p(cos.data_ptr()),
            C.c_void_p(sin.data_ptr()), pid, C.c_longlong(B * S), S, int(pos_offset), C.c_void_p(_lib.stream())),
            "qkv_norm_rope_fwd")
        ctx.save_for_backward(qkv, stats, f[0], f[2], cos, sin, pos_ids if pos_ids is not None else cos.new_empty(0))
        ctx.meta = (hq, hkv, pos_offset, pos_ids is not None, [t.dtype for t in (gq, bq, gk, bk)])
        return out[:, :, :hq], out[:, :, hq:hq + hkv], out[:, :, hq + hkv:]

    @staticmethod
    def backward(ctx, dq, dk, dv):
        qkv, stats, gq, gk, cos, sin, pos_ids = ctx.saved_tensors
        hq, hkv, pos_offset, has_ids, dtypes = ctx.meta
        B, S, W = qkv.shape
        hd = 128
        fixed = []
        for g, h in ((dq, hq), (dk, hkv), (dv, hkv)):
            if g is None:
                g = torch.zeros((B, S, h, hd), device=qkv.device, dtype=torch.bfloat16)
            if g.stride(3) != 1 or g.stride(0) != S * g.stride(1) or g.stride(1) % 8 or g.stride(2) % 8:
                g = g.contiguous()
            fixed.append(g)
        dq, dk, dv = fixed
        lib = _lib.lib()
        T = B * S
        dqkv = torch.empty((B, S, W), device=qkv.device, dtype=qkv.dtype)
        dparams = torch.empty((4, hd), device=qkv.device, dtype=torch.float32)
        scratch = torch.empty((lib.np_qkv_norm_rope_parts(C.c_longlong(T)), 4 * hd), device=qkv.device,
                              dtype=torch.float32)
        _lib.check(lib.np_qkv_norm_rope_bwd(
            C.c_void_p(dq.data_ptr()), C.c_longlong(dq.stride(1)), C.c_longlong(dq.stride(2)),
            C.c_void_p(dk.data_ptr()), C.c_longlong(dk.stride(1)), C.c_longlong(dk.stride(2)),
            C.c_void_p(dv.data_ptr()), C.c_longlong(dv.stride(1)), C.c_longlong(dv.stride(2)),
            C.c_void_p(qkv.data_ptr()), C.c_longlong(qkv.stride(1)), hq, hkv, C.c_void_p(gq.data_ptr()),
            C.c_void_p(gk.data_ptr()), C.c_void_p(stats.data_ptr()), C.c_void_p(dqkv.data_ptr()),
            C.c_void_p(dparams.data_ptr()), C.c_void_p(scratch.data_ptr()), C.c_void_p(cos.data_ptr()),
            C.c_void_p(sin.data_ptr()), C.c_void_p(pos_ids.data_ptr() if has_ids else 0), C.c_longlong(T), S,
            int(pos_offset), 0, C.c_void_p(_lib.stream())), "qkv_norm_rope_bwd")
        dgq, dbq, dgk, dbk = [dparams[i].to(dt) for i, dt in enumerate(dtypes)]
        return dqkv, dgq, dbq, dgk, dbk, None, None, None, None, None, None, None


def qkv_norm_rope_supported(qkv: torch.Tensor, cos, hq: int, hkv: int, hd: int) -> bool:
    S = qkv.shape[1]
    return (_lib.on(qkv) and qkv.dtype == torch.bfloat16 and hd == 128 and cos.shape[1] == 64 and
            cos.dtype == torch.float32 and qkv.stride(2) == 1 and qkv.stride(1) % 8 == 0 and
            qkv.stride(0) == S * qkv.stride(1) and (hq + hkv) * 8 <= 512 and (hq + hkv) * 8 + hkv * 16 <= 768)


def qkv_norm_rope(qkv, q_norm, k_norm, cos, sin, hq: int, hkv: int, pos_offset: int = 0, pos_ids=None):
    """``qkv [B, S, (hq+2*hkv)*128]`` -> LayerNorm'ed and rotated ``q``, ``k`` and ``v`` (views of one buffer);
    ``q_norm`` / ``k_norm`` are the ``nn.LayerNorm(128)`` modules of the attention layer."""
    if pos_ids is not None:
        pos_ids = pos_ids.reshape(-1).to(torch.int32)
    return _QKVNormRope.apply(qkv, q_norm.weight, q_norm.bias, k_norm.weight, k_norm.bias, float(q_norm.eps), cos, sin,
                              hq, hkv, pos_offset, pos_ids)


def qkv_rope(qkv: torch.Tensor, cos, sin, hq: int, hkv: int, hd: int, pos_offset: int = 0, pos_ids=None):
    """``qkv [B, S, (hq+2*hkv)*hd]`` -> rotated ``q [B,S,hq,hd]``, ``k [B,S,hkv,hd]`` and ``v`` (strided views of
    one buffer). Falls back to slicing + ``apply_rope`` off the kernel path."""
    B, S, W = qkv.shape
    ok = (_lib.on(qkv) and qkv.dtype == torch.bfloat16 and hd % 8 == 0 and (2 * cos.shape[1]) % 16 == 0 and
          qkv.stride(2) == 1 and qkv.stride(1) % 8 == 0 and qkv.stride(0) == S * qkv.stride(1) and
          cos.dtype == torch.float32)
    if ok:
        if pos_ids is not None:
            pos_ids = pos_ids.reshape(-1).to(torch.int32)
        return _QKVRope.apply(qkv, cos, sin, hq, hkv, hd, pos_offset, pos_ids)
    q = qkv[..., : hq * hd].unflatten(-1, (hq, hd))
    k = qkv[..., hq * hd:(hq + hkv) * hd].unflatten(-1, (hkv, hd))
    v = qkv[..., (hq + hkv) * hd:].unflatten(-1, (hkv, hd))
    return apply_rope(q, cos, sin, pos_offset, pos_ids), apply_rope(k, cos, sin, pos_offset, pos_ids), v
