"""MXFP8 (1x32 power-of-two scales) quantiser and GEMM: the PyTorch statements that the sm_100a kernels are tested
against, checked here against plain fp32 math."""
import torch

from nanopysche_b200.ops.gemm_mxfp8 import (gemm_mxfp8, mx_dequantize, mx_quantize, sf_bytes, sf_index)


def test_scale_layout_is_a_bijection_onto_the_chunks():
    rows, K = 384, 512
    idx = sf_index(rows, K).reshape(-1)
    assert idx.unique().numel() == idx.numel() == rows * K // 32
    assert int(idx.max()) < sf_bytes(rows, K) == (rows // 128) * (K // 128) * 512
    # row 33, 32-block 5 -> chunk 0 * 4 + 1, lane 1, word 1, byte 1
    assert int(sf_index(rows, K)[33, 5]) == 1 * 512 + 1 * 16 + 1 * 4 + 1
    # row 200 (block 1, r = 72: lane 8, word 2), 32-block 14 (chunk 3, byte 2)
    assert int(sf_index(rows, K)[200, 14]) == (1 * 4 + 3) * 512 + 8 * 16 + 2 * 4 + 2


def test_quantise_round_trip_error_and_scale_choice():
    torch.manual_seed(0)
    x = (torch.randn(200, 256) * torch.logspace(-4, 4, 200).view(-1, 1)).bfloat16()
    x[7] = 0
    q, sf = mx_quantize(x)
    assert q.dtype == torch.float8_e4m3fn and sf.dtype == torch.uint8 and sf.numel() == sf_bytes(200, 256)
    d = mx_dequantize(q, sf)
    blocks = x.float().view(200, 8, 32)
    err = (d.view(200, 8, 32) - blocks).abs().amax(-1)
    assert bool((err <= blocks.abs().amax(-1) * 2 ** -4 + 1e-30).all())   # 3 mantissa bits, no saturation
    assert bool((d[7] == 0).all())
    e = sf[sf_index(200, 256).reshape(-1)].view(200, 8).float() - 127
    am = blocks.abs().amax(-1)
    nz = am > 0
    assert bool((am[nz] / torch.exp2(e[nz]) <= 448).all()) and bool((am[nz] / torch.exp2(e[nz]) > 224).all())


def test_gemm_reference_tracks_fp32_matmul():
    torch.manual_seed(1)
    a, b = torch.randn(256, 384).bfloat16(), torch.randn(128, 384).bfloat16()
    aq, sa = mx_quantize(a)
    bq, sb = mx_quantize(b)
    y = gemm_mxfp8(aq, sa, bq, sb, out_dtype=torch.float32)
    ref = a.float() @ b.float().t()
    assert float((y - ref).norm() / ref.norm()) < 0.06
    grp = torch.tensor([0, 0], dtype=torch.int32)
    yg = gemm_mxfp8(aq, sa, bq, sb, out_dtype=torch.float32, mblk_group=grp, rows_per_group=128)
    assert torch.allclose(yg, y, rtol=1e-4, atol=1e-3)
