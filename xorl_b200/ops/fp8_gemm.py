"""Block-scaled fp8 GEMM dispatch: tcgen05 kernel on CUDA (``csrc/quant.cu``), reference elsewhere."""
from __future__ import annotations

import torch

from . import _lib
from . import quantize as Q

_launches = 0


def launch_count() -> int:
    return _launches


def block_fp8_gemm(a_q, a_s, b_q, b_s, out_dtype=torch.bfloat16):
    """C[M,N] = sum_kb (A_kb B_kb^T) * a_s[m,kb] * b_s[n/128,kb]; A [M,K] e4m3 with 1x128 scales,
    B [N,K] e4m3 with 128x128 scales."""
    global _launches
    lib = _lib.cuda_lib() if (a_q.is_cuda and _lib.have_cuda_lib()) else None
    if lib is not None and hasattr(lib, "xb_block_fp8_gemm") and out_dtype == torch.bfloat16 \
            and a_q.shape[1] % 128 == 0:
        M, K = a_q.shape
        N = b_q.shape[0]
        out = torch.empty((M, N), device=a_q.device, dtype=torch.bfloat16)
        a_s = a_s.float().contiguous()
        b_s = b_s.float().contiguous()
        lib.xb_block_fp8_gemm.restype = _lib.c_int
        rc = lib.xb_block_fp8_gemm(_lib.P(a_q.data_ptr()), _lib.P(b_q.data_ptr()), _lib.P(out.data_ptr()),
                                   _lib.P(a_s.data_ptr()), _lib.P(b_s.data_ptr()), _lib.I(M), _lib.I(N),
                                   _lib.I(K), _lib.P(_lib.stream_ptr()))
        _lib.check(rc, "xb_block_fp8_gemm")
        _launches += 1
        return out
    return Q.block_fp8_gemm_reference(a_q, a_s, b_q, b_s, out_dtype=out_dtype)
