"""AdamW with decoupled weight decay (reference: optim/adamw.py:24-162).

``AdamW`` is a ``torch.optim.Optimizer`` with the reference's update rule and state names; on CUDA
fp32 parameters each tensor is updated by the fused sm_100a kernel (one launch per tensor, no
foreach temporaries). Whole-model training on B200 uses ``optim.arena.ArenaAdamW`` instead, which
updates one flat buffer per step. ``create_adamw`` builds the decay / no-decay groups; its no-decay
rule is "bias, norm, embedding, or any tensor with fewer than 2 dims" (the reference's predicate
has an operator-precedence slip that makes the last clause a no-op).
"""
from __future__ import annotations

import torch
from torch.optim import Optimizer

from ..ops import _lib


class AdamW(Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas: tuple[float, float] = (0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.01, amsgrad: bool = False):
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay, amsgrad=amsgrad))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, (b1, b2), eps, wd = group["lr"], group["betas"], group["eps"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("AdamW does not support sparse gradients")
                st = self.state[p]
                if len(st) == 0:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p)
                    st["exp_avg_sq"] = torch.zeros_like(p)
                    if group["amsgrad"]:
                        st["max_exp_avg_sq"] = torch.zeros_like(p)
                st["step"] += 1
                m, v = st["exp_avg"], st["exp_avg_sq"]
                fused = (p.is_cuda and p.dtype == torch.float32 and p.grad.dtype == torch.float32 and
                         p.is_contiguous() and p.grad.is_contiguous() and not group["amsgrad"])
                if fused:
                    _lib.call("adamw", p, p.grad, m, v, None, _lib.LL(p.numel()), float(lr), float(b1), float(b2),
                              float(eps), float(wd), int(st["step"]), None, None)
                    continue
                g = p.grad
                if wd > 0:
                    p.mul_(1 - lr * wd)
                m.mul_(b1).add_(g, alpha=1 - b1)
                v.mul_(b2).addcmul_(g, g, value=1 - b2)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                if group["amsgrad"]:
                    torch.max(st["max_exp_avg_sq"], v, out=st["max_exp_avg_sq"])
                    denom = (st["max_exp_avg_sq"].sqrt() / (bc2 ** 0.5)).add_(eps)
                else:
                    denom = (v.sqrt() / (bc2 ** 0.5)).add_(eps)
                p.addcdiv_(m, denom, value=-lr / bc1)
        return loss


def is_no_decay(name: str, param: torch.Tensor) -> bool:
    return "bias" in name or "norm" in name or "emb" in name or param.dim() < 2


def create_adamw(model: torch.nn.Module, lr: float = 3e-4, weight_decay: float = 0.1,
                 betas: tuple[float, float] = (0.9, 0.95)) -> AdamW:
    decay, no_decay = [], []
    for name, p in model.named_parameters():
        if p.requires_grad:
            (no_decay if is_no_decay(name, p) else decay).append(p)
    return AdamW([{"params": decay, "weight_decay": weight_decay}, {"params": no_decay, "weight_decay": 0.0}],
                 lr=lr, betas=betas)
