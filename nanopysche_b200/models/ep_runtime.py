"""Host-side EP runtime heuristics (reference: model/moe.py:716-1156, same class and method names).

``AdaptiveSMAllocator`` decides how many SMs the dispatch / combine kernels may take from the expert GEMMs,
``RoutingPrefetcher`` predicts next-step routing from history and ``CoupledEPScheduler`` couples the SM split, the
prefetch confidence and the re-balancing strength to the measured load imbalance. Pure host arithmetic.

The SM split is not the reference's proportional rule (SMs in the ratio of communication time to total time, with
H100 constants and a per-token compute time against a whole-batch transfer time). On a B200 the two kernels run side
by side, so the layer takes ``max(t_comm(s), t_gemm(148 - s))``; a pushing SM sustains only a share of the NVLink
port, which saturates at 770 GB/s (measured, per direction) - after about sixteen SMs by this model's estimate of 48
GB/s per SM, a figure that has not been measured on its own - and the GEMM's rate is proportional to the SMs it keeps. The allocator returns the ``s`` that minimises that maximum: the smallest budget that
hides the transfer under the GEMM when that is possible, the saturation point when it is not.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class _LinkComputeModel:
    """Seconds for an expert-parallel exchange and for the expert GEMMs of one layer as functions of the SM split."""

    total_sms: int = 148
    link_gbps: float = 770.0          # measured peer-copy bandwidth per direction (nominal 900)
    per_sm_gbps: float = 48.0         # estimate of what one SM of 16-byte peer stores sustains (port full near 16 SMs)
    tflops: float = 1590.0            # measured cuBLAS bf16 burst rate of the whole GPU (nominal 2250 dense)

    def t_comm(self, nbytes: float, sms: int) -> float:
        return nbytes / (min(sms * self.per_sm_gbps, self.link_gbps) * 1e9)

    def t_gemm(self, flops: float, sms: int) -> float:
        return flops / (self.tflops * 1e12 * max(sms, 1) / self.total_sms)

    def best_split(self, nbytes: float, flops: float, lo: int, hi: int) -> int:
        """``s`` in ``[lo, hi]`` minimising ``max(t_comm(s), t_gemm(total - s))``; ties go to the smaller budget."""
        best, best_t = lo, float("inf")
        for s in range(lo, hi + 1):
            t = max(self.t_comm(nbytes, s), self.t_gemm(flops, self.total_sms - s))
            if t < best_t - 1e-15:
                best, best_t = s, t
        return best


class AdaptiveSMAllocator:
    # nominal figures kept as class attributes for callers that read them (the reference's names)
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
        # the achievable rates scale with the nominal ones the caller gave (770 / 900 and 1590 / 2250 measured on B200)
        self.model = _LinkComputeModel(total_sms=self.TOTAL_SMS, link_gbps=self.NVLINK_BW_GBPS * 770.0 / 900.0,
                                       tflops=self.GPU_TFLOPS_BF16 * 1590.0 / 2250.0)
        self._ema_alpha = 0.3
        self._ema_bytes: Optional[float] = None
        self._ema_flops: Optional[float] = None

    def _smooth(self, nbytes: float, flops: float) -> tuple:
        """Exponential average of the workload over calls: the split should not jump with one odd batch."""
        a = self._ema_alpha
        self._ema_bytes = nbytes if self._ema_bytes is None else a * nbytes + (1 - a) * self._ema_bytes
        self._ema_flops = flops if self._ema_flops is None else a * flops + (1 - a) * self._ema_flops
        return self._ema_bytes, self._ema_flops

    def compute_optimal_sms(self, num_tokens: int, hidden_size: int, expert_hidden: int, num_experts: int,
                            num_topk: int, num_bytes_per_elem: int = 2) -> int:
        """SM budget of the dispatch / combine kernels for a layer that moves ``num_tokens x num_topk`` rows of
        ``hidden_size`` elements and runs three ``hidden_size x expert_hidden`` GEMMs on each of them."""
        rows = num_tokens * num_topk
        if rows <= 0:
            return self.min_sms
        nbytes, flops = self._smooth(rows * hidden_size * num_bytes_per_elem,
                                     rows * 6.0 * hidden_size * expert_hidden)
        return self.model.best_split(nbytes, flops, self.min_sms, self.max_sms)

    def compute_optimal_sms_from_counts(self, tokens_per_expert: torch.Tensor, hidden_size: int,
                                        expert_hidden: int, num_bytes_per_elem: int = 2) -> int:
        """The same from measured per-expert loads. An uneven load makes the busiest expert's rows the critical path of
        both kernels; the transfer of those rows cannot be spread over more links, so the budget grows with the
        imbalance (up to one half more) to start the longest GEMM earlier."""
        total = float(tokens_per_expert.sum().item())
        if total == 0:
            return self.min_sms
        n = tokens_per_expert.shape[0]
        spread = (tokens_per_expert.float() * n / total).std().item() if n > 1 else 0.0
        base = self.compute_optimal_sms(int(total), hidden_size, expert_hidden, n, 1, num_bytes_per_elem)
        return max(self.min_sms, min(self.max_sms, int(base * (1.0 + min(0.5, 0.1 * spread)))))


class RoutingPrefetcher:
    """Predicts where a layer's tokens will be routed from where they went in the last few steps, so that a runtime
    may start moving rows before the router has run (reference: model/moe.py ``RoutingPrefetcher``, same methods).

    Per layer the last ``history_len`` index tensors sit in one ring buffer ``[history_len, tokens, K]``. A prediction
    is each token position's expert with the largest *recency-weighted* vote (every step counts twice as much as the
    one before it: routing drifts, so older steps together never outvote the newest one, they only decide between its
    K experts); its confidence is that expert's share of the weighted votes, i.e. how long it has been chosen."""

    def __init__(self, num_experts: int, history_len: int = 4, confidence_threshold: float = 0.8,
                 max_prefetch_tokens: int = 4096):
        self.num_experts = num_experts
        self.history_len = history_len
        self.confidence_threshold = confidence_threshold
        self.max_prefetch_tokens = max_prefetch_tokens
        self._ring: dict[int, torch.Tensor] = {}      # layer -> [history_len, tokens, K] int64
        self._filled: dict[int, int] = {}             # layer -> number of steps recorded (saturates at history_len)
        self._hit_count = 0
        self._miss_count = 0

    def record_routing(self, layer_idx: int, expert_indices: torch.Tensor):
        idx = expert_indices.detach().to("cpu", torch.int64)
        flat = idx.reshape(-1, idx.shape[-1])
        ring = self._ring.get(layer_idx)
        if ring is None or ring.shape[1:] != flat.shape:       # first step, or the batch shape changed: start over
            ring = torch.zeros((self.history_len, *flat.shape), dtype=torch.int64)
            self._ring[layer_idx], self._filled[layer_idx] = ring, 0
        ring.copy_(torch.roll(ring, shifts=-1, dims=0))         # oldest step out, newest into the last slot
        ring[-1] = flat
        self._filled[layer_idx] = min(self._filled[layer_idx] + 1, self.history_len)

    def should_prefetch(self, layer_idx: int) -> bool:
        return self._filled.get(layer_idx, 0) >= 2

    def predict_next_layer(self, layer_idx: int, current_indices: torch.Tensor):
        """``(predicted (B, S, K), confident (B, S))`` or ``None`` before two steps are known. Every one of the K slots
        carries the same predicted expert (the most voted one)."""
        if not self.should_prefetch(layer_idx):
            return None
        B, S, K = current_indices.shape
        n = self._filled[layer_idx]
        ring = self._ring[layer_idx][-n:]
        if ring.shape[1] != B * S:
            return None
        weights = (2.0 ** torch.arange(n, dtype=torch.float32)).view(n, 1, 1).expand(n, B * S, ring.shape[2])
        votes = torch.zeros(B * S, self.num_experts)
        votes.scatter_add_(1, ring.permute(1, 0, 2).reshape(B * S, -1), weights.permute(1, 0, 2).reshape(B * S, -1))
        share, expert = (votes / votes.sum(-1, keepdim=True).clamp_min(1.0)).max(dim=-1)
        # an expert chosen in every remembered step by one of K slots has a share of 1 / K: compare on that scale
        confident = (share * K).clamp(max=1.0) >= self.confidence_threshold
        return expert.view(B, S, 1).expand(B, S, K), confident.view(B, S)

    def record_outcome(self, predicted: torch.Tensor, actual: torch.Tensor, mask: Optional[torch.Tensor] = None):
        """Score a prediction against the routing that happened (feeds ``get_stats``)."""
        hit = (predicted[..., :1].cpu() == actual.cpu()).any(-1)
        if mask is not None:
            hit = hit[mask.cpu()]
        self._hit_count += int(hit.sum())
        self._miss_count += int(hit.numel() - hit.sum())

    def get_stats(self) -> dict:
        total = self._hit_count + self._miss_count
        return {"hit_rate": self._hit_count / max(1, total), "total_predictions": total,
                "hits": self._hit_count, "misses": self._miss_count,
                "history_depth": dict(self._filled)}

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
    """One decision per step from the measured per-expert loads: the imbalance (coefficient of variation, smoothed)
    drives the SM budget of the exchange (the allocator's balanced split, widened with the imbalance), how much a
    routing prediction is trusted, how hard the router's bias should push back, and whether the exchange may use the
    fixed-capacity fast path."""

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
        self._allocator = AdaptiveSMAllocator(total_sms, nvlink_bw_gbps, gpu_tflops_bf16, min_sms=min_sms)
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
        cv = self._ema_cv
        balanced = self._allocator.compute_optimal_sms(num_tokens, self.hidden_size, self.expert_hidden,
                                                       self.num_experts, num_topk)
        sms = min(self.total_sms - 4, max(self.min_sms, int(balanced * (1.0 + min(1.0, cv)))))
        return EPScheduleDecision(
            num_sms=sms,
            prefetch_confidence=max(0.1, min(0.95, 1.0 - 0.8 * cv)),      # skewed routing changes faster
            load_rebalancing_strength=min(0.9, max(0.1, 0.8 * cv)),
            imbalance_coefficient=cv,
            dispatch_mode="fast" if cv < 0.3 else "safe",
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
