"""Host-side EP runtime heuristics (reference: model/moe.py:716-1156).

``AdaptiveSMAllocator`` splits SMs between the dispatch/combine kernels and the expert GEMMs from a
roofline estimate, ``RoutingPrefetcher`` predicts next-step routing from history and
``CoupledEPScheduler`` couples SM split, prefetch confidence and re-balancing strength to the
measured imbalance. Pure host arithmetic; the defaults here are B200 figures (148 SMs, 900 GB/s per
direction of NVLink 5, 2250 dense bf16 TFLOP/s) instead of the reference's H100 ones, and the
per-token compute time is multiplied by the token count so both terms of the roofline are seconds
for the whole batch (the reference compares whole-batch communication with per-token compute).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


class AdaptiveSMAllocator:
    NVLINK_BW_GBPS: float = 900.0
    GPU_TFLOPS_BF16: float = 2250.0
    TOTAL_SMS: int = 148

    def __init__(self, total_sms: Optional[int] = None, nvlink_bw_gbps: Optional[float] = None,
                 gpu_tflops: Optional[float] = None, min_sms: int = 4, max_sms: Optional[int] = None):
        if total_sms is not None:
            self.TOTAL_SMS = total_sms
        if nvlink_bw_gbps is not None:
            self.NVLINK_BW_GBPS = nvlink_bw_gbps
        if gpu_tflops is not None:
            self.GPU_TFLOPS_BF16 = gpu_tflops
        self.min_sms = min_sms
        self.max_sms = max_sms or (self.TOTAL_SMS - 4)
        self._prev_comm_time = 0.0
        self._prev_compute_time = 0.0
        self._ema_alpha = 0.3

    def compute_optimal_sms(self, num_tokens: int, hidden_size: int, expert_hidden: int, num_experts: int,
                            num_topk: int, num_bytes_per_elem: int = 2) -> int:
        comm_bytes = num_tokens * num_topk * hidden_size * num_bytes_per_elem
        comm_time = comm_bytes / (self.NVLINK_BW_GBPS * 1e9)
        flops = num_tokens * num_topk * (2 * hidden_size * expert_hidden * 3)
        compute_time = flops / (self.GPU_TFLOPS_BF16 * 1e12)
        a = self._ema_alpha
        comm_time = a * comm_time + (1 - a) * self._prev_comm_time
        compute_time = a * compute_time + (1 - a) * self._prev_compute_time
        self._prev_comm_time, self._prev_compute_time = comm_time, compute_time
        total = comm_time + compute_time
        if total == 0:
            return self.min_sms
        return max(self.min_sms, min(self.max_sms, int(self.TOTAL_SMS * comm_time / total)))

    def compute_optimal_sms_from_counts(self, tokens_per_expert: torch.Tensor, hidden_size: int,
                                        expert_hidden: int, num_bytes_per_elem: int = 2) -> int:
        num_experts = tokens_per_expert.shape[0]
        total_tokens = float(tokens_per_expert.sum().item())
        if total_tokens == 0:
            return self.min_sms
        mean_tokens = total_tokens / num_experts
        imbalance = (tokens_per_expert.float() / mean_tokens).std().item() if num_experts > 1 else 0.0
        base = self.compute_optimal_sms(int(total_tokens), hidden_size, expert_hidden, num_experts, 1,
                                        num_bytes_per_elem)
        boosted = int(base * (1.0 + min(0.5, imbalance * 0.1)))
        return max(self.min_sms, min(self.max_sms, boosted))


class RoutingPrefetcher:
    def __init__(self, num_experts: int, history_len: int = 4, confidence_threshold: float = 0.8,
                 max_prefetch_tokens: int = 4096):
        self.num_experts = num_experts
        self.history_len = history_len
        self.confidence_threshold = confidence_threshold
        self.max_prefetch_tokens = max_prefetch_tokens
        self._routing_history: dict[int, list[torch.Tensor]] = {}
        self._prefetch_cache: dict[int, torch.Tensor] = {}
        self._hit_count = 0
        self._miss_count = 0

    def record_routing(self, layer_idx: int, expert_indices: torch.Tensor):
        hist = self._routing_history.setdefault(layer_idx, [])
        hist.append(expert_indices.detach().cpu())
        if len(hist) > self.history_len:
            hist.pop(0)

    def predict_next_layer(self, layer_idx: int, current_indices: torch.Tensor):
        history = self._routing_history.get(layer_idx, [])
        if len(history) < 2:
            return None
        stacked = torch.stack(history[-self.history_len:], dim=0)  # (H, B, S, K)
        B, S, K = current_indices.shape
        flat = stacked.reshape(stacked.shape[0], B * S, K).permute(1, 0, 2).reshape(B * S, -1).long()
        counts = torch.zeros(B * S, self.num_experts, dtype=torch.float32)
        counts.scatter_add_(1, flat, torch.ones_like(flat, dtype=torch.float32))
        probs = counts / counts.sum(-1, keepdim=True).clamp(min=1)
        confidence, predicted = probs.max(dim=-1)
        predicted = predicted.reshape(B, S, 1).expand(B, S, K)
        confident = confidence.reshape(B, S) >= self.confidence_threshold
        return predicted, confident

    def record_outcome(self, predicted: torch.Tensor, actual: torch.Tensor, mask: Optional[torch.Tensor] = None):
        """Score a prediction against the routing that happened (feeds ``get_stats``)."""
        hit = (predicted[..., :1].cpu() == actual.cpu()).any(-1)
        if mask is not None:
            hit = hit[mask.cpu()]
        self._hit_count += int(hit.sum())
        self._miss_count += int(hit.numel() - hit.sum())

    def should_prefetch(self, layer_idx: int) -> bool:
        return len(self._routing_history.get(layer_idx, [])) >= 2

    def get_stats(self) -> dict:
        total = self._hit_count + self._miss_count
        return {"hit_rate": self._hit_count / max(1, total), "total_predictions": total,
                "hits": self._hit_count, "misses": self._miss_count,
                "history_depth": {k: len(v) for k, v in self._routing_history.items()}}

    def reset_stats(self):
        self._hit_count = 0
        self._miss_count = 0


@dataclass
class EPScheduleDecision:
    num_sms: int
    prefetch_confidence: float
    load_rebalancing_strength: float
    imbalance_coefficient: float
    dispatch_mode: str


class CoupledEPScheduler:
    def __init__(self, num_experts: int, hidden_size: int, expert_hidden: int, total_sms: int = 148,
                 nvlink_bw_gbps: float = 900.0, gpu_tflops_bf16: float = 2250.0, ema_alpha: float = 0.3,
                 min_sms: int = 4):
        self.num_experts = num_experts
        self.hidden_size = hidden_size
        self.expert_hidden = expert_hidden
        self.total_sms = total_sms
        self.nvlink_bw_gbps = nvlink_bw_gbps
        self.gpu_tflops_bf16 = gpu_tflops_bf16
        self.ema_alpha = ema_alpha
        self.min_sms = min_sms
        self._ema_cv = 0.0
        self._step_count = 0
        self._routing_history: list[torch.Tensor] = []
        self._history_len = 4

    def schedule(self, tokens_per_expert: torch.Tensor, num_tokens: int, num_topk: int) -> EPScheduleDecision:
        if num_tokens == 0 or float(tokens_per_expert.sum()) == 0:
            return EPScheduleDecision(self.min_sms, 0.5, 0.0, 0.0, "safe")
        t = tokens_per_expert.float()
        cv = (t.std() / (t.mean() + 1e-8)).item() if t.numel() > 1 else 0.0
        self._ema_cv = self.ema_alpha * cv + (1 - self.ema_alpha) * self._ema_cv
        self._step_count += 1
        comm_fraction = min(1.0, self._ema_cv * 1.5)
        base = max(self.min_sms, int(self.total_sms * comm_fraction * 0.5))
        sms = min(self.total_sms - 4, max(self.min_sms, base))
        return EPScheduleDecision(
            num_sms=sms,
            prefetch_confidence=max(0.1, min(0.95, 1.0 - self._ema_cv * 0.8)),
            load_rebalancing_strength=min(0.9, max(0.1, self._ema_cv * 0.8)),
            imbalance_coefficient=self._ema_cv,
            dispatch_mode="fast" if self._ema_cv < 0.3 else "safe",
        )

    def update_routing_history(self, expert_indices: torch.Tensor):
        self._routing_history.append(expert_indices.detach().cpu())
        if len(self._routing_history) > self._history_len:
            self._routing_history.pop(0)

    def predict_next_layer(self) -> Optional[torch.Tensor]:
        return self._routing_history[-1] if len(self._routing_history) >= 2 else None

    def get_state(self) -> dict:
        return {"ema_cv": self._ema_cv, "step_count": self._step_count}

    def load_state(self, state: dict):
        self._ema_cv = state.get("ema_cv", 0.0)
        self._step_count = state.get("step_count", 0)
