"""Causal / full softmax attention, GQA-native.

Layout is ``[B, S, H, hd]`` (heads contiguous after the QKV GEMM); K/V keep their ``Hkv`` heads -
the reference's ``repeat_interleave`` expansion (model/attention.py:166-169) is never materialised.
Returns the log-sum-exp as well when asked, which the context-parallel ring uses to merge partial
results (the reference sums per-chunk softmax outputs with no LSE merge,
distributed/context_parallel.py:307-317).

Single-device attention currently goes through PyTorch SDPA (a library flash kernel on CUDA); the
chunked LSE form below is the oracle and the CPU path for ring attention.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


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


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              attn_mask: torch.Tensor | None = None, scale: float | None = None) -> torch.Tensor:
    """``softmax(q k^T / sqrt(hd)) v`` for ``q [B,S,Hq,hd]``, ``k/v [B,Sk,Hkv,hd]`` -> ``[B,S,Hq,hd]``."""
    Hq, Hkv = q.shape[2], k.shape[2]
    qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    is_causal = causal and attn_mask is None and q.shape[1] == k.shape[1]
    if causal and not is_causal and attn_mask is None:
        # decode / kv-cache: query i sits at position Sk - Sq + i
        Sq, Sk = q.shape[1], k.shape[1]
        attn_mask = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device).tril(diagonal=Sk - Sq)
    o = F.scaled_dot_product_attention(qt, kt, vt, attn_mask=attn_mask, is_causal=is_causal, scale=scale,
                                       enable_gqa=(Hq != Hkv))
    return o.transpose(1, 2)
