"""Tokens dropped by the capacity rule under skewed routing (the reference's table "Token Dropping Under Skewed
Routing", train/README.md:56-70: 8 experts, top-2, 8192 tokens, experts 0 and 1 drawing five times the traffic of the
others, capacity factors 1.0 .. 4.0 and dropless).

    python -m benchmarks.token_dropping [--tokens 8192] [--experts 8] [--top-k 2] [--skew 5] [--device cpu]

Two figures per capacity factor: the sum of the per-expert overflows, which is what the reference's table counts (a
token is counted once per over-full expert it chose, hence rates above 100 %), and the number of tokens that lose their
MoE output (a token over capacity at any of its experts is dropped whole). The routing is synthetic - every token
draws its top-k experts without replacement, the two hot experts with ``skew`` times the weight of the others - so
only the capacity arithmetic is exercised. (The script behind the reference's table is not part of its tree, so its
draw cannot be matched; the two definitions are what carries over.)"""
from __future__ import annotations

import argparse
import json
import math

import torch


def run(tokens: int, experts: int, top_k: int, skew: float, device: str, seed: int = 0):
    from nanopysche_b200.models.moe import MoEBase

    g = torch.Generator().manual_seed(seed)
    logits = torch.zeros(tokens, experts)
    logits[:, :2] += math.log(skew)
    # top-k without replacement with probabilities proportional to exp(logits): the Gumbel-top-k draw
    gumbel = -torch.log(-torch.log(torch.rand(tokens, experts, generator=g).clamp_min(1e-20)))
    idx = (logits + gumbel).topk(top_k, dim=-1).indices.to(device)
    w = torch.full((tokens, top_k), 1.0 / top_k, device=device)
    x = torch.zeros(tokens, 8, device=device)
    rows = []
    for cf in (1.0, 1.25, 1.5, 2.0, 4.0, None):
        moe = MoEBase(d_model=8, hidden_size=256, num_experts=experts, top_k=top_k, capacity_factor=cf)
        if cf is None:
            rows.append({"capacity_factor": "dropless", "overflow_slots": 0, "overflow_rate_pct": 0.0,
                         "tokens_dropped": 0, "token_drop_rate_pct": 0.0})
            continue
        moe._apply_capacity(x, w, idx)
        slots, toks = moe.last_dropped_slots, int(moe.last_dropped)
        rows.append({"capacity_factor": cf, "overflow_slots": slots, "overflow_rate_pct": 100.0 * slots / tokens,
                     "tokens_dropped": toks, "token_drop_rate_pct": 100.0 * toks / tokens})
    return rows


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--top-k", type=int, default=2)
    ap.add_argument("--skew", type=float, default=5.0)
    ap.add_argument("--device", default="cpu")
    args = ap.parse_args()
    for r in run(args.tokens, args.experts, args.top_k, args.skew, args.device):
        print(json.dumps(r))


if __name__ == "__main__":
    main()
