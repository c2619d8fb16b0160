"""Causal / full softmax attention, GQA-native.

Layout is ``[B, S, H, hd]`` (heads contiguous after the QKV GEMM); K/V keep their ``Hkv`` heads -
the reference's ``repeat_interleave`` expansion (model/attention.py:166-169) is never materialised.
Returns the log-sum-exp as well when asked, which the context-parallel ring uses to merge partial
results (the reference sums per-chunk softmax outputs with no LSE merge,
distributed/context_parallel.py:307-317).

On bf16 CUDA tensors with head_dim 128 attention runs on this library's tcgen05 flash kernels
(csrc/attn_sm100.cu: forward, dQ and dK/dV kernels; scores, probabilities and the output accumulator live
in tensor memory); other shapes and the CPU use PyTorch SDPA. The explicit-position fp32 form below is the
oracle of the kernels and the CPU path of ring attention.
"""
from __future__ import annotations

import math

import torch
import os

import torch.nn.functional as F

from . import _lib

# Limit of every in-kernel wait of the multi-GPU paths (default 10 s); on expiry the kernel reports through the
# library status word and returns.
WAIT_LIMIT_NS = int(float(os.environ.get("NPB200_WAIT_LIMIT_MS", "10000")) * 1e6)
# Single-device attention runs on the tcgen05 flash kernels whenever they cover the case; NPB200_SDPA=1 routes it
# through PyTorch SDPA instead.
USE_FLASH = os.environ.get("NPB200_SDPA", "0") != "1"
PAD_SMALL_HEADS = os.environ.get("NPB200_PAD_SMALL_HEADS", "1") == "1"   # head_dim < 128 on the flash kernels, padded


def attention_ref(q, k, v, causal=True, q_pos=None, k_pos=None, scale=None):
    """fp32 reference with explicit positions; returns (out [B,S,H,hd], lse [B,H,S]).

    ``q_pos`` / ``k_pos`` ([Sq] / [Sk] global positions) define the causal mask ``k_pos <= q_pos`` so
    sharded sequences (zig-zag chunks) mask correctly. Rows with no visible key give out=0, lse=-inf.
    """
    B, Sq, Hq, hd = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    scale = scale or 1.0 / math.sqrt(hd)
    qf = q.float().permute(0, 2, 1, 3)
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    s = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        qp = torch.arange(Sq, device=q.device) + (Sk - Sq) if q_pos is None else q_pos
        kp = torch.arange(Sk, device=q.device) if k_pos is None else k_pos
        mask = kp[None, :] <= qp[:, None]
        s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    p = torch.exp(s - lse.clamp_min(-1e30).unsqueeze(-1))
    p = torch.where(torch.isfinite(lse).unsqueeze(-1), p, torch.zeros_like(p))
    o = (p @ vf).permute(0, 2, 1, 3)
    return o.to(q.dtype), lse


def merge_attention(o1, lse1, o2, lse2):
    """Combine two partial attention results over disjoint key sets (online-softmax merge)."""
    lse = torch.logaddexp(lse1, lse2)
    w1 = torch.exp(lse1 - lse).nan_to_num(0.0)
    w2 = torch.exp(lse2 - lse).nan_to_num(0.0)
    w1 = w1.permute(0, 2, 1).unsqueeze(-1)
    w2 = w2.permute(0, 2, 1).unsqueeze(-1)
    o = o1.float() * w1 + o2.float() * w2
    return o.to(o1.dtype), lse


def _strides3(t: torch.Tensor):
    assert t.stride(3) == 1, "head_dim must be contiguous"
    return t.stride(0), t.stride(1), t.stride(2)


def _set_flags(a, flags, keep: list):
    """``flags``: None, or a dict ``flags`` (int32 tensor), ``idx`` (flag index per source), ``epoch``, ``epoch_base``
    (device counter tensor) [, ``which``] naming sources that peers are still pushing into local memory."""
    import ctypes as C

    if not flags:
        return
    idx = (C.c_int * len(flags["idx"]))(*[int(i) for i in flags["idx"]])
    keep.append(idx)
    a.src_flags, a.flag_idx = flags["flags"].data_ptr(), C.cast(idx, C.c_void_p)
    a.flag_epoch, a.epoch_base, a.flag_limit_ns = int(flags["epoch"]), flags["epoch_base"].data_ptr(), WAIT_LIMIT_NS
    if hasattr(a, "flag_which"):
        a.flag_which = int(flags.get("which", 3))
    a.flag_own = int(flags.get("own", -1)) + 1
    push = flags.get("push")
    if push:   # dict k, v (contiguous shards), dst / flag (lists of peer addresses), ctr (zeroed [2] int32 tensor)
        n = len(push["dst"])
        dst = (C.c_void_p * n)(*[int(x) for x in push["dst"]])
        flg = (C.c_void_p * n)(*[int(x) for x in push["flag"]])
        keep += [dst, flg]
        a.push_k, a.push_v = push["k"].data_ptr(), push["v"].data_ptr()
        a.push_bytes, a.push_n = push["k"].numel() * push["k"].element_size(), n
        a.push_dst, a.push_flag = C.cast(dst, C.c_void_p), C.cast(flg, C.c_void_p)
        a.push_ctr = push["ctr"].data_ptr()


def flash_supported(q: torch.Tensor, k: torch.Tensor) -> bool:
    """The tcgen05 kernels cover bf16, head_dim 128, 16-byte aligned strided ``[B, S, H, 128]`` views."""
    return (_lib.on(q) and q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and q.shape[-1] == 128
            and k.shape[-1] == 128 and q.stride(-1) == 1 and k.stride(-1) == 1 and _lib.available()
            and all(s % 8 == 0 for s in q.stride()[:3]) and all(s % 8 == 0 for s in k.stride()[:3]))


def flash_fwd(q, k_list, v_list, *, causal=True, scale=None, q_off=0, q_blk_pos=None, k_blk_pos=None, split=0,
              flags=None):
    """Forward flash attention on the tcgen05 kernel. ``k_list`` / ``v_list`` are lists of equally shaped
    ``[B, Sk, Hkv, 128]`` KV sources (one entry without context parallelism; one per rank's shard - any of
    them may live in a peer's memory - with it). Returns ``(out [B,Sq,Hq,128] bf16, lse [B,Hq,Sq] fp32)``."""
    import ctypes as C

    if not isinstance(k_list, (list, tuple)):
        k_list, v_list = [k_list], [v_list]
    B, Sq, Hq, hd = q.shape
    k_ref = next(t for t in k_list if isinstance(t, torch.Tensor))   # peers may be given as raw device pointers
    Sk, Hkv = k_ref.shape[1], k_ref.shape[2]
    n = len(k_list)
    o = torch.empty((B, Sq, Hq, hd), device=q.device, dtype=torch.bfloat16)
    lse = torch.empty((B, Hq, Sq), device=q.device, dtype=torch.float32)
    a = _lib.AttnFwdArgs()
    a.q = q.data_ptr()
    a.q_sb, a.q_ss, a.q_sh = _strides3(q)
    kp = (C.c_void_p * n)(*[t.data_ptr() if isinstance(t, torch.Tensor) else int(t) for t in k_list])
    vp = (C.c_void_p * n)(*[t.data_ptr() if isinstance(t, torch.Tensor) else int(t) for t in v_list])
    a.k_ptrs, a.v_ptrs = C.cast(kp, C.c_void_p), C.cast(vp, C.c_void_p)
    a.k_sb, a.k_ss, a.k_sh = _strides3(k_ref)
    a.o = o.data_ptr()
    a.o_sb, a.o_ss, a.o_sh = _strides3(o)
    a.lse = lse.data_ptr()
    a.B, a.Sq, a.Hq, a.Hkv, a.causal, a.n_src, a.src_len, a.q_off = B, Sq, Hq, Hkv, int(causal), n, Sk, q_off
    a.scale = scale or 1.0 / math.sqrt(hd)
    a.q_blk_pos = q_blk_pos.data_ptr() if q_blk_pos is not None else None
    a.k_blk_pos = k_blk_pos.data_ptr() if k_blk_pos is not None else None
    a.split = split
    keep = []
    _set_flags(a, flags, keep)
    _lib.check(_lib.lib().np_attn_fwd(C.byref(a), C.c_void_p(_lib.stream())), "attn_fwd")
    return o, lse


def _ptr_array(items):
    import ctypes as C

    arr = (C.c_void_p * len(items))(*[t.data_ptr() if isinstance(t, torch.Tensor) else int(t) for t in items])
    return arr, C.cast(arr, C.c_void_p)


def flash_bwd(q, k, v, o, d_o, lse, *, causal=True, scale=None, q_off=0, delta=None, sources=None, phase=3, split=0,
              flags=None, skip=0, out=None,
              q_blk_pos_local=None, k_blk_pos_all=None, k_blk_pos_local=None, q_blk_pos_all=None):
    """Backward of ``flash_fwd``: returns ``(dq, dk, dv)`` in bf16 with the shapes of q / k / v.

    ``sources`` (context parallelism) is a dict of equally long lists ``k, v, q, d_o, lse, delta`` holding one
    tensor (or raw device pointer into a peer's memory) per rank of the group; the local tensors are used
    when it is ``None``. ``phase=1`` only computes ``delta`` (so that it can be published to the peers
    before ``phase=2`` runs the dQ and dK/dV kernels)."""
    import ctypes as C

    B, Sq, Hq, hd = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    if delta is None:
        delta = torch.empty((B, Hq, Sq), device=q.device, dtype=torch.float32)
    if d_o.stride(3) != 1 or any(s % 8 for s in d_o.stride()[:3]):
        d_o = d_o.contiguous()
    # ``out``: optional (dq, dk, dv) destinations (tensors or raw device pointers, layouts of q / k); ``skip``:
    # 1 = no dQ kernel, 2 = no dK/dV kernel
    dq = dk = dv = None
    if phase & 2:
        if out is not None:
            dq, dk, dv = out
        else:
            dq = torch.empty((B, Sq, Hq, hd), device=q.device, dtype=torch.bfloat16) if not skip & 1 else None
            dk = torch.empty((B, Sk, Hkv, hd), device=q.device, dtype=torch.bfloat16) if not skip & 2 else None
            dv = torch.empty_like(dk) if not skip & 2 else None
    a = _lib.AttnBwdArgs()
    a.q, a.k, a.v, a.o, a.d_o = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr()
    a.q_sb, a.q_ss, a.q_sh = _strides3(q)
    a.k_sb, a.k_ss, a.k_sh = _strides3(k)
    assert _strides3(v) == _strides3(k), "k and v must share their strides"
    a.o_sb, a.o_ss, a.o_sh = _strides3(o)
    a.do_sb, a.do_ss, a.do_sh = _strides3(d_o)
    a.lse, a.delta = lse.data_ptr(), delta.data_ptr()
    if phase & 2:
        ptr = lambda t: None if t is None else (t.data_ptr() if isinstance(t, torch.Tensor) else int(t))  # noqa: E731
        a.dq, a.dk, a.dv = ptr(dq), ptr(dk), ptr(dv)
        a.dq_sb, a.dq_ss, a.dq_sh = _strides3(dq) if isinstance(dq, torch.Tensor) else (Sq * Hq * hd, Hq * hd, hd)
        a.dk_sb, a.dk_ss, a.dk_sh = _strides3(dk) if isinstance(dk, torch.Tensor) else (Sk * Hkv * hd, Hkv * hd, hd)
    # source lists: missing entries default to the local tensors, short lists are padded to the longest one
    defaults = dict(k=k, v=v, q=q, d_o=d_o, lse=lse, delta=delta)
    src = dict(sources) if sources else {}
    n_src = max([len(src.get(nm) or []) for nm in defaults] + [1])
    for nm, dflt in defaults.items():
        lst = [dflt if t is None else t for t in (src.get(nm) or [dflt])]
        src[nm] = lst + [lst[0]] * (n_src - len(lst))
    keep = [_ptr_array(src[n]) for n in ("k", "v", "q", "d_o", "lse", "delta")]
    a.k_src, a.v_src, a.q_src, a.do_src, a.lse_src, a.delta_src = [x[1] for x in keep]
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.causal, a.n_src, a.q_off, a.phase = \
        B, Sq, Sk, Hq, Hkv, int(causal), n_src, q_off, phase
    a.scale = scale or 1.0 / math.sqrt(hd)
    a.split, a.skip = split, skip
    _set_flags(a, flags, keep)
    for name, t in (("q_blk_pos_local", q_blk_pos_local), ("k_blk_pos_all", k_blk_pos_all),
                    ("k_blk_pos_local", k_blk_pos_local), ("q_blk_pos_all", q_blk_pos_all)):
        setattr(a, name, t.data_ptr() if t is not None else None)
    _lib.check(_lib.lib().np_attn_bwd(C.byref(a), C.c_void_p(_lib.stream())), "attn_bwd")
    return dq, dk, dv, delta


def flash_fwd_raw(q_ptr, k_ptrs, v_ptrs, o_ptr, lse_ptr, *, like_q, like_k, heads, lse_heads, causal=True, scale=None,
                  q_blk_pos=None, k_blk_pos=None, like_o=None, flags=None):
    """``flash_fwd`` on raw device pointers (any of them may point into a peer's memory). The tensors have the
    shapes and strides of ``like_q`` / ``like_k`` except for the head count, which is ``heads = (Hq, Hkv)``: a launch
    can cover a head slice of larger buffers. The output and the log-sum-exp are stored through ``o_ptr`` /
    ``lse_ptr`` (layout of ``like_q`` and ``[B, lse_heads, Sq]``)."""
    import ctypes as C

    B, Sq, _, hd = like_q.shape
    a = _lib.AttnFwdArgs()
    a.q, a.o, a.lse = int(q_ptr), int(o_ptr), int(lse_ptr)
    a.q_sb, a.q_ss, a.q_sh = _strides3(like_q)
    a.o_sb, a.o_ss, a.o_sh = _strides3(like_o if like_o is not None else like_q)
    a.k_sb, a.k_ss, a.k_sh = _strides3(like_k)
    kk, vv = _ptr_array(k_ptrs), _ptr_array(v_ptrs)
    a.k_ptrs, a.v_ptrs = kk[1], vv[1]
    a.B, a.Sq, a.Hq, a.Hkv, a.causal, a.n_src, a.src_len, a.q_off = \
        B, Sq, heads[0], heads[1], int(causal), len(k_ptrs), like_k.shape[1], 0
    a.scale = scale or 1.0 / math.sqrt(hd)
    a.q_blk_pos = q_blk_pos.data_ptr() if q_blk_pos is not None else None
    a.k_blk_pos = k_blk_pos.data_ptr() if k_blk_pos is not None else None
    a.lse_heads = lse_heads
    keep = []
    _set_flags(a, flags, keep)
    _lib.check(_lib.lib().np_attn_fwd(C.byref(a), C.c_void_p(_lib.stream())), "attn_fwd")


def flash_bwd_raw(ptr, src, *, lse, delta, like_q, like_k, heads, lse_heads, causal=True, scale=None, blk_local=None,
                  blk_all=None, like_dq=None, like_dk=None, flags=None):
    """dQ and dK/dV kernels on raw device pointers. ``ptr``: dict ``q, d_o, k, v, dq, dk, dv`` of the tensors this
    launch owns (inputs of the layouts of ``like_q`` / ``like_k`` with ``heads = (Hq, Hkv)`` heads; the gradients
    are stored through ``dq / dk / dv``); ``src``: dict of per-rank pointer lists ``k, v, q, d_o, lse, delta``."""
    import ctypes as C

    B, Sq, _, hd = like_q.shape
    a = _lib.AttnBwdArgs()
    a.q, a.d_o, a.k, a.v = int(ptr["q"]), int(ptr["d_o"]), int(ptr["k"]), int(ptr["v"])
    a.dq, a.dk, a.dv = int(ptr["dq"]), int(ptr["dk"]), int(ptr["dv"])
    a.lse, a.delta = int(lse), int(delta)
    a.q_sb, a.q_ss, a.q_sh = _strides3(like_q)
    a.do_sb, a.do_ss, a.do_sh = _strides3(like_q)
    a.dq_sb, a.dq_ss, a.dq_sh = _strides3(like_dq if like_dq is not None else like_q)
    a.k_sb, a.k_ss, a.k_sh = _strides3(like_k)
    a.dk_sb, a.dk_ss, a.dk_sh = _strides3(like_dk if like_dk is not None else like_k)
    keep = [_ptr_array(src[n]) for n in ("k", "v", "q", "d_o", "lse", "delta")]
    a.k_src, a.v_src, a.q_src, a.do_src, a.lse_src, a.delta_src = [x[1] for x in keep]
    a.B, a.Sq, a.Sk, a.Hq, a.Hkv, a.causal, a.n_src, a.q_off, a.phase = \
        B, Sq, like_k.shape[1], heads[0], heads[1], int(causal), len(src["k"]), 0, 2
    a.scale = scale or 1.0 / math.sqrt(hd)
    a.lse_heads = lse_heads
    a.q_blk_pos_local = a.k_blk_pos_local = blk_local.data_ptr() if blk_local is not None else None
    a.k_blk_pos_all = a.q_blk_pos_all = blk_all.data_ptr() if blk_all is not None else None
    _set_flags(a, flags, keep)
    _lib.check(_lib.lib().np_attn_bwd(C.byref(a), C.c_void_p(_lib.stream())), "attn_bwd")


class _FlashAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale):
        o, lse = flash_fwd(q, k, v, causal=causal, scale=scale, q_off=(k.shape[1] - q.shape[1]) if causal else 0)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.causal, ctx.scale = causal, scale
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv, _ = flash_bwd(q, k, v, o, d_o, lse, causal=ctx.causal, scale=ctx.scale,
                                  q_off=(k.shape[1] - q.shape[1]) if ctx.causal else 0)
        return dq, dk, dv, None, None


def flash_attention(q, k, v, causal=True, scale=None):
    """Differentiable attention on the tcgen05 flash kernels (see ``flash_supported``)."""
    if k.stride() != v.stride():
        v = v.contiguous() if k.is_contiguous() else v
        if k.stride() != v.stride():
            k, v = k.contiguous(), v.contiguous()
    return _FlashAttention.apply(q, k, v, causal, scale)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              attn_mask: torch.Tensor | None = None, scale: float | None = None) -> torch.Tensor:
    """``softmax(q k^T / sqrt(hd)) v`` for ``q [B,S,Hq,hd]``, ``k/v [B,Sk,Hkv,hd]`` -> ``[B,S,Hq,hd]``."""
    Hq, Hkv = q.shape[2], k.shape[2]
    if USE_FLASH and attn_mask is None and flash_supported(q, k) and (not causal or q.shape[1] <= k.shape[1]):
        return flash_attention(q, k, v, causal=causal, scale=scale)
    hd = q.shape[-1]
    if USE_FLASH and PAD_SMALL_HEADS and attn_mask is None and _lib.on(q) and q.dtype == torch.bfloat16 and \
            k.dtype == torch.bfloat16 and hd < 128 and hd % 8 == 0 and (not causal or q.shape[1] <= k.shape[1]):
        # head dims below 128 (the 125m / 350m / 1b presets have 64): zero-pad the head dimension so the tcgen05
        # kernels apply. The padded columns add nothing to q.k and come out of P.V as zeros; the price is the work
        # of the padding (twice the FLOPs and traffic at 64). ``NPB200_SDPA=1`` picks PyTorch's library kernel instead.
        pad = (0, 128 - hd)
        o = flash_attention(F.pad(q, pad), F.pad(k, pad), F.pad(v, pad), causal=causal,
                            scale=scale if scale is not None else 1.0 / math.sqrt(hd))
        return o[..., :hd]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    is_causal = causal and attn_mask is None and q.shape[1] == k.shape[1]
    if causal and not is_causal and attn_mask is None:
        # decode / kv-cache: query i sits at position Sk - Sq + i
        Sq, Sk = q.shape[1], k.shape[1]
        attn_mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril(diagonal=Sk - Sq)
    o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=attn_mask, is_causal=is_causal, scale=scale,
                                       enable_gqa=(Hq != Hkv))
    return o.transpose(1, 2)
