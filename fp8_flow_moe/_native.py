"""Binding of this package's sm_100a kernels (used when a GPU is present).

The package stays importable and fully functional without them: every operator has a PyTorch path. Lookup order:
``FP8_FLOW_MOE_LIB``; the training framework's library when this package sits next to ``nanopysche_b200`` (it links
the same sources, so one library is loaded per process); this package's own ``lib/libfp8flow.so``, built from
``csrc/`` on first use when nvcc is there (``python -m fp8_flow_moe.build``).
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

import torch

_NATIVE = None


class _Native:
    def __init__(self, lib):
        self.lib = lib

    @staticmethod
    def _stream():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def _check(self, rc, name):
        if rc != 0:
            raise RuntimeError(f"{name} failed with code {rc}")

    def quant_1x128(self, x):
        rows, cols = x.numel() // x.shape[-1], x.shape[-1]
        q = torch.empty(x.shape, device=x.device, dtype=torch.float8_e4m3fn)
        s = torch.empty((*x.shape[:-1], cols // 128), device=x.device, dtype=torch.float32)
        self._check(self.lib.np_quant_1x128(C.c_void_p(x.data_ptr()), C.c_void_p(q.data_ptr()),
                                            C.c_void_p(s.data_ptr()), C.c_longlong(rows), C.c_longlong(cols),
                                            self._stream()), "quant_1x128")
        return q, s

    def swiglu_quant(self, gate, up):
        rows, cols = gate.numel() // gate.shape[-1], gate.shape[-1]
        q = torch.empty(gate.shape, device=gate.device, dtype=torch.float8_e4m3fn)
        s = torch.empty((*gate.shape[:-1], cols // 128), device=gate.device, dtype=torch.float32)
        self._check(self.lib.np_swiglu_quant(C.c_void_p(gate.data_ptr()), C.c_void_p(up.data_ptr()),
                                             C.c_void_p(q.data_ptr()), C.c_void_p(s.data_ptr()), C.c_longlong(rows),
                                             C.c_longlong(cols), C.c_longlong(gate.stride(-2) if gate.dim() > 1 else 0),
                                             C.c_longlong(up.stride(-2) if up.dim() > 1 else 0), self._stream()),
                    "swiglu_quant")
        return q, s

    def dequant_1x128(self, q, s):
        rows, cols = q.numel() // q.shape[-1], q.shape[-1]
        out = torch.empty(q.shape, device=q.device, dtype=torch.bfloat16)
        self._check(self.lib.np_dequant_1x128(C.c_void_p(q.data_ptr()), C.c_void_p(s.contiguous().data_ptr()),
                                              C.c_void_p(out.data_ptr()), C.c_longlong(rows), C.c_longlong(cols),
                                              self._stream()), "dequant_1x128")
        return out

    def quant_128x128(self, w):
        R, Cc = w.shape
        q = torch.empty(w.shape, device=w.device, dtype=torch.float8_e4m3fn)
        s = torch.empty((R // 128, Cc // 128), device=w.device, dtype=torch.float32)
        self._check(self.lib.np_quant_128x128(C.c_void_p(w.data_ptr()), C.c_void_p(q.data_ptr()),
                                              C.c_void_p(s.data_ptr()), R, Cc, self._stream()), "quant_128x128")
        return q, s

    def transpose_1x128(self, q, s):
        M, N = q.shape
        qt = torch.empty((N, M), device=q.device, dtype=torch.float8_e4m3fn)
        st = torch.empty((N, M // 128), device=q.device, dtype=torch.float32)
        self._check(self.lib.np_transpose_1x128(C.c_void_p(q.data_ptr()), C.c_void_p(s.contiguous().data_ptr()),
                                                C.c_void_p(qt.data_ptr()), C.c_void_p(st.data_ptr()), M, N,
                                                self._stream()), "transpose_1x128")
        return qt, st


    def expert_rank(self, indices, num_experts, pad_multiple):
        n = indices.numel()
        idx = indices.reshape(-1).to(torch.int64).contiguous()
        row_map = torch.empty(n, device=idx.device, dtype=torch.int64)
        padded = torch.empty(num_experts, device=idx.device, dtype=torch.int64)
        self._check(self.lib.np_expert_rank(C.c_void_p(idx.data_ptr()), n, num_experts, pad_multiple,
                                            C.c_void_p(row_map.data_ptr()), C.c_void_p(padded.data_ptr()),
                                            self._stream()), "expert_rank")
        return row_map, padded

    def move_rows(self, x, out, row_map, weights, scatter):
        w = weights.reshape(-1).float().contiguous() if weights is not None else None
        self._check(self.lib.np_move_rows(C.c_void_p(x.data_ptr()), C.c_void_p(out.data_ptr()),
                                          C.c_void_p(row_map.data_ptr()), C.c_void_p(w.data_ptr() if w is not None else 0),
                                          C.c_longlong(row_map.numel()), C.c_longlong(x.shape[1] * x.element_size()),
                                          int(scatter), self._stream()), "move_rows")
        return out


def native():
    global _NATIVE
    if _NATIVE is None:
        here = Path(__file__).resolve().parent
        cand = os.environ.get("FP8_FLOW_MOE_LIB")
        if not cand:
            sibling = here.parent / "nanopysche_b200" / "lib" / "libnpb200.so"
            if sibling.exists():
                cand = str(sibling)
            else:
                own = here / "lib" / "libfp8flow.so"
                if not own.exists():
                    from .build import build_extension

                    build_extension()
                cand = str(own)
        _NATIVE = _Native(C.CDLL(cand))
    return _NATIVE
