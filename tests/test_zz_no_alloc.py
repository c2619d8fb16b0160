"""The allocation-free RMSNorm backward (``np_rmsnorm_bwd_noalloc``).

Some users of the kernel library cannot allocate device memory at the point of the call - a stream
under capture, a latency-critical loop that must stay out of the allocator, a host application with a
fixed memory budget - so this entry point keeps its scratch in a static device array inside the
library. The test calls it through its exported C symbol, twice in a row (the scratch keeps the first
call's contents, so the second call proves nothing stale is read), and compares every output with the
regular entry point, which takes a caller-provided scratch buffer.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run_both(lib, rows, cols, accumulate, seed):
    torch.manual_seed(seed)
    dev = "cuda"
    dy = torch.randn(rows, cols, device=dev).bfloat16()
    x = torch.randn(rows, cols, device=dev).bfloat16()
    dres = torch.randn(rows, cols, device=dev).bfloat16()
    w = torch.rand(cols, device=dev) + 0.5
    rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-6).contiguous()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: C.c_void_p(t.data_ptr())  # noqa: E731
    # regular entry point: caller-provided scratch
    parts = lib.np_rmsnorm_bwd_parts(rows)
    scratch = torch.empty(parts, cols, device=dev)
    dx_ref = torch.empty_like(x)
    dw_ref = torch.full((cols,), 0.25, device=dev)
    rc = lib.np_rmsnorm_bwd(p(dy), p(x), p(w), p(rstd), p(dres), p(dx_ref), p(dw_ref), p(scratch), rows, cols,
                            accumulate, stream)
    assert rc == 0
    # allocation-free entry point
    dx = torch.empty_like(x)
    dw = torch.full((cols,), 0.25, device=dev)
    before = torch.cuda.memory_allocated()
    rc = lib.np_rmsnorm_bwd_noalloc(p(dy), p(x), p(w), p(rstd), p(dres), p(dx), p(dw), rows, cols, accumulate, stream)
    assert rc == 0
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    assert torch.equal(dx, dx_ref)
    assert torch.allclose(dw, dw_ref, rtol=1e-6, atol=1e-6)
    # and both agree with plain PyTorch fp32 math
    xf, dyf = x.float(), dy.float()
    xhat = xf * rstd[:, None]
    g = dyf * w
    dx_t = rstd[:, None] * (g - xhat * (g * xhat).mean(-1, keepdim=True)) + dres.float()
    dw_t = (dyf * xhat).sum(0) + (0.25 if accumulate else 0.0)
    assert ((dx.float() - dx_t).norm() / dx_t.norm()).item() < 8e-3
    assert ((dw - dw_t).norm() / dw_t.norm()).item() < 1e-4


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    from nanopysche_b200.ops import _lib

    lib = _lib.lib()
    lib.np_rmsnorm_bwd_noalloc.restype = C.c_int
    # two calls in a row with different shapes and contents share the static scratch
    _run_both(lib, rows=1000, cols=2048, accumulate=0, seed=1)
    _run_both(lib, rows=37, cols=4096, accumulate=1, seed=2)
    _run_both(lib, rows=1000, cols=2048, accumulate=0, seed=3)


def test_noalloc_rejects_sizes_beyond_the_static_scratch():
    from nanopysche_b200.ops import _lib

    lib = _lib.lib()
    t = torch.zeros(8, 8192, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8192, device="cuda")
    p = lambda a: C.c_void_p(a.data_ptr())  # noqa: E731
    rc = lib.np_rmsnorm_bwd_noalloc(p(t), p(t), p(f), p(f), None, p(t), p(f), 8, 8192, 0,
                                    C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 3
