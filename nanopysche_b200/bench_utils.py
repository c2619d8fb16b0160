"""Peak-FLOPs tables, model FLOPs estimate and MFU (reference: bench_utils.py:35-209).

Same function signatures. The B200 rows hold the dense tensor-core peaks (2.25 PFLOP/s bf16,
4.5 fp8) rather than half of the fp8 figure, and the MoE term counts ``top_k`` active experts per
token (the reference multiplies by ``top_k / num_experts`` of one expert, which under-counts).
"""
from __future__ import annotations

import logging
from typing import Optional

import torch

PEAK_FLOPS = {"A100": 312e12, "A10G": 125e12, "A10": 125e12, "H100": 989e12, "H200": 989e12, "B200": 2250e12,
              "L4": 121e12, "T4": 65e12, "V100": 125e12}
FP8_PEAK_FLOPS = {"A100": 624e12, "H100": 1979e12, "H200": 1979e12, "B200": 4500e12}


def _gpu_key(device: Optional[torch.device], table: dict) -> Optional[str]:
    if not torch.cuda.is_available():
        return None
    name = torch.cuda.get_device_name(device if device is not None and torch.device(device).type == "cuda" else 0)
    for k in sorted(table, key=len, reverse=True):
        if k in name:
            return k
    return None


def has_fp8_tensor_cores(device: Optional[torch.device] = None) -> bool:
    if not torch.cuda.is_available():
        return False
    major, minor = torch.cuda.get_device_capability(device if device is not None and
                                                    torch.device(device).type == "cuda" else 0)
    return (major, minor) >= (8, 9)


def get_peak_flops(device: Optional[torch.device] = None, fp8: bool = False) -> float:
    """Dense peak of the device; 0.0 for anything that is not a CUDA device, which makes ``compute_mfu`` report 0
    there (reference: bench_utils.py:72-103)."""
    if not torch.cuda.is_available() or (device is not None and torch.device(device).type != "cuda"):
        return 0.0
    table = FP8_PEAK_FLOPS if fp8 else PEAK_FLOPS
    k = _gpu_key(device, table)
    if k is None:
        return PEAK_FLOPS["A100"]
    return table[k]


def estimate_model_flops(n_layers: int, d_model: int, ffn_hidden: int, n_heads: int, seq_len: int, batch_size: int,
                         num_experts: int = 0, top_k: int = 0, reference_moe_count: bool = False) -> float:
    """FLOPs of one forward+backward pass: per token per layer ``8 d^2 + 4 S d`` (attention) plus
    ``6 d h`` per active MLP, times 3 for forward+backward."""
    tokens = batch_size * seq_len
    attn = (8 * d_model * d_model + 4 * seq_len * d_model) * n_layers
    mlp = 6 * d_model * ffn_hidden
    if num_experts > 0 and top_k > 0:
        mlp = mlp * (top_k / num_experts if reference_moe_count else top_k)
    mlp *= n_layers
    fwd = (attn + mlp) * tokens + 2 * d_model * tokens
    return 3.0 * fwd


def compute_mfu(step_time_seconds: float, n_layers: int, d_model: int, ffn_hidden: int, n_heads: int, seq_len: int,
                batch_size: int, device: Optional[torch.device] = None, fp8: bool = False, num_gpus: int = 1,
                num_experts: int = 0, top_k: int = 0) -> float:
    actual_fp8 = fp8 and has_fp8_tensor_cores(device)
    if fp8 and not actual_fp8:
        logging.getLogger("bench_utils").warning("FP8 requested but no FP8 tensor cores; using the bf16 peak")
    peak = get_peak_flops(device, fp8=actual_fp8) * num_gpus
    if peak <= 0 or step_time_seconds <= 0:
        return 0.0
    flops = estimate_model_flops(n_layers, d_model, ffn_hidden, n_heads, seq_len, batch_size, num_experts, top_k)
    return flops / step_time_seconds / peak
