"""DiLoCo-style gradient compressor (reference: optim/diko.py:21-145).

Random-sign chunk-sum projection of the flat gradient to ``compression_rank`` numbers with error
feedback; only the projected vector is all-reduced. The projection is one segmented reduction
(``reshape + sum``) instead of the reference's Python loop over chunks, and the shared random signs
come from a private generator (the reference reseeds the global RNG in its constructor).

Error feedback keeps the residual ``(gradient + previous residual) - reconstruction`` for the next step. The
reference's ``decompress`` subtracts the reconstruction from the old buffer without adding the gradient
(optim/diko.py:112-113), so its buffer never sees what the projection dropped; a ``decompress`` call that was not
preceded by ``compress`` keeps that behaviour.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


class DiLoCoCompressor:
    def __init__(self, params, compression_rank: int = 256, group=None, seed: int = 42):
        params = list(params)
        self.compression_rank = compression_rank
        self.group = group
        self.total_params = sum(p.numel() for p in params)
        self.device = params[0].device if params else torch.device("cpu")
        gen = torch.Generator(device="cpu").manual_seed(seed)
        self._random_diag = torch.randn(self.total_params, generator=gen).to(self.device)
        self.error_buffer = torch.zeros(self.total_params, device=self.device)
        self._pending = None      # gradient + residual of the compress() call that a decompress() has not yet closed

    def _chunks(self, n: int):
        chunk = max(1, n // self.compression_rank)
        head = chunk * (self.compression_rank - 1)
        return chunk, min(head, n)

    def _fast_project(self, g: torch.Tensor, direction: str = "forward") -> torch.Tensor:
        gs = g * self._random_diag[: g.shape[0]]
        chunk, head = self._chunks(g.shape[0])
        proj = torch.zeros(self.compression_rank, device=g.device, dtype=g.dtype)
        rows = head // chunk
        if rows:
            proj[:rows] = gs[:head].reshape(rows, chunk).sum(1)
        proj[rows] = gs[head:].sum()
        return proj / (g.shape[0] ** 0.5)

    def _fast_reconstruct(self, v: torch.Tensor, N: int) -> torch.Tensor:
        chunk, head = self._chunks(N)
        rows = head // chunk
        rec = torch.empty(N, device=v.device, dtype=v.dtype)
        if rows:
            rec[:head] = (v[:rows] / chunk).repeat_interleave(chunk)
        rec[head:] = v[rows] / chunk
        return rec * self._random_diag[:N]

    def compress(self, gradients: torch.Tensor):
        g = gradients + self.error_buffer[: gradients.shape[0]]
        self._pending = g
        compressed = self._fast_project(g)
        return compressed, compressed.abs().max().clamp(min=1e-8)

    def decompress(self, compressed: torch.Tensor, scale: torch.Tensor, N: int) -> torch.Tensor:
        rec = self._fast_reconstruct(compressed, N)
        if self._pending is not None and self._pending.shape[0] == N:
            self.error_buffer[:N] = self._pending - rec
        else:
            self.error_buffer[:N] = self.error_buffer[:N] - rec
        self._pending = None
        return rec

    def all_reduce_gradients(self, gradients: torch.Tensor) -> torch.Tensor:
        N = gradients.shape[0]
        compressed, scale = self.compress(gradients)
        if dist.is_available() and dist.is_initialized():
            dist.all_reduce(compressed, op=dist.ReduceOp.SUM, group=self.group)
            compressed = compressed / dist.get_world_size(self.group)
        return self.decompress(compressed, scale, N)

    def compress_state_dict(self, state_dict: dict) -> dict:
        flat = torch.cat([g.reshape(-1).float() for g in state_dict.values()])
        compressed, scale = self.compress(flat)
        return {"compressed": compressed, "scale": scale, "total_params": flat.shape[0],
                "shapes": {k: v.shape for k, v in state_dict.items()}}
