"""Block-scaled fp8 GEMM and its quantisers: tcgen05 ``kind::f8f6f4`` kernel with per-K-block scale
promotion on CUDA (``csrc/quant.cu``), the dequantise-and-matmul reference elsewhere."""
from __future__ import annotations

import torch

from . import _lib
from . import quantize as Q

_launches = 0


def launch_count() -> int:
    return _launches


def _on_device(t: torch.Tensor) -> bool:
    return t.is_cuda and _lib.have_cuda_lib()


def quantize_rows(x: torch.Tensor):
    """bf16 [M,K] -> (e4m3 [M,K], fp32 scales [M,K/128]); K a multiple of 128."""
    global _launches
    if _on_device(x) and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 128 == 0:
        x = x.contiguous()
        M, K = x.shape
        q = torch.empty((M, K), device=x.device, dtype=torch.float8_e4m3fn)
        s = torch.empty((M, K // 128), device=x.device, dtype=torch.float32)
        _lib.check(_lib.cuda_lib().xb_quant_fp8_rows(x.data_ptr(), K, q.data_ptr(), K, s.data_ptr(), K // 128,
                                                     M, K, _lib.stream_ptr()), "xb_quant_fp8_rows")
        _launches += 1
        return q, s
    return Q.block_fp8_quantize_1x128(x)


def quantize_blocks(w: torch.Tensor):
    """bf16 [N,K] -> (e4m3 [N,K], fp32 scales [ceil(N/128), ceil(K/128)])."""
    global _launches
    if _on_device(w) and w.dtype == torch.bfloat16 and w.dim() == 2:
        w = w.contiguous()
        N, K = w.shape
        q = torch.empty((N, K), device=w.device, dtype=torch.float8_e4m3fn)
        s = torch.empty(((N + 127) // 128, (K + 127) // 128), device=w.device, dtype=torch.float32)
        _lib.check(_lib.cuda_lib().xb_quant_fp8_blocks(w.data_ptr(), K, q.data_ptr(), K, s.data_ptr(),
                                                       s.shape[1], N, K, _lib.stream_ptr()), "xb_quant_fp8_blocks")
        _launches += 1
        return q, s
    return Q.block_fp8_quantize_128x128(w)


def dequantize_blocks(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    global _launches
    if _on_device(q) and q.dim() == 2:
        q = q.contiguous()
        s = s.float().contiguous()
        N, K = q.shape
        w = torch.empty((N, K), device=q.device, dtype=torch.bfloat16)
        _lib.check(_lib.cuda_lib().xb_dequant_fp8_blocks(q.data_ptr(), K, s.data_ptr(), s.shape[1], w.data_ptr(),
                                                         K, N, K, _lib.stream_ptr()), "xb_dequant_fp8_blocks")
        _launches += 1
        return w
    return Q.block_fp8_dequantize_128x128(q, s)


def block_fp8_gemm(a_q, a_s, b_q, b_s, out_dtype=torch.bfloat16):
    """C[M,N] = sum_kb (A_kb B_kb^T) * a_s[m,kb] * b_s[n/128,kb]; A [M,K] e4m3 with 1x128 scales,
    B [N,K] e4m3 with 128x128 scales."""
    global _launches
    if _on_device(a_q) and out_dtype == torch.bfloat16 and a_q.shape[1] % 128 == 0:
        a_q, b_q = a_q.contiguous(), b_q.contiguous()
        M, K = a_q.shape
        N = b_q.shape[0]
        out = torch.empty((M, N), device=a_q.device, dtype=torch.bfloat16)
        a_s = a_s.float().contiguous()
        b_s = b_s.float().contiguous()
        rc = _lib.cuda_lib().xb_block_fp8_gemm_ex(a_q.data_ptr(), b_q.data_ptr(), out.data_ptr(), a_s.data_ptr(),
                                                  b_s.data_ptr(), M, N, K, K, K, N, a_s.shape[1], b_s.shape[1],
                                                  _lib.stream_ptr())
        _lib.check(rc, "xb_block_fp8_gemm")
        _launches += 1
        return out
    return Q.block_fp8_gemm_reference(a_q, a_s, b_q, b_s, out_dtype=out_dtype)
