"""Quantisation codecs: round-trip error bounds and the block-fp8 GEMM scheme."""
import pytest
import torch

from xorl_b200.ops import quantize as Q


@pytest.mark.parametrize("fmt,group,tol", [("nf4", 64, 0.12), ("int4", 128, 0.12), ("nvfp4", 16, 0.15),
                                           ("mxfp4", 32, 0.3), ("block_fp8", 128, 0.05)])
def test_roundtrip(fmt, group, tol):
    torch.manual_seed(0)
    w = torch.randn(256, 384) * 0.05
    parts = Q.quantize_weight(w, fmt, group)
    back = Q.dequantize_weight(parts, fmt, group, w.shape, torch.float32)
    rel = (back - w).norm() / w.norm()
    assert rel < tol, (fmt, rel)
    assert parts["packed"].dtype == torch.uint8


def test_block_fp8_gemm_scheme():
    torch.manual_seed(0)
    a, b = torch.randn(64, 256), torch.randn(192, 256)
    aq, as_ = Q.block_fp8_quantize_1x128(a)
    bq, bs = Q.block_fp8_quantize_128x128(b)
    assert as_.shape == (64, 2) and bs.shape == (2, 2)
    c = Q.block_fp8_gemm_reference(aq, as_, bq, bs, out_dtype=torch.float32)
    ref = a @ b.t()
    assert (c - ref).norm() / ref.norm() < 0.06
