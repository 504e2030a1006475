"""Causal depthwise convolution over packed documents and 4-bit weight dequantisation
(``csrc/seqmix.cu``).

``causal_conv1d(x, weight, bias, cu_seqlens, silu)`` is the short convolution in front of the
GatedDeltaNet and Mamba2 recurrences: ``y[t, c] = act(bias[c] + sum_j w[c, j] * x[t-(K-1)+j, c])``
with taps that never reach across a document start
(src/xorl/ops/linear_attention/ops/causal_conv1d_triton.py:24, src/xorl/ops/ssm/conv.py).
On a GPU with bf16 inputs the CUDA kernels run (forward; backward = dpre, dx and per-chunk
dw / dbias partial sums added in a fixed order); elsewhere the same arithmetic runs as tensor ops.

``dequant4(parts, fmt, group, shape)`` decodes NF4 / INT4 / NVFP4 / MXFP4 packed weights to bf16
on the device (src/xorl/ops/quantize/*_quantize.py)."""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn.functional as F

from . import _lib

_launches = 0

MAX_TAPS = 8
_FMT_CODE = {"nf4": 0, "int4": 1, "nvfp4": 2, "mxfp4": 3}


def launch_count() -> int:
    return _launches


def document_starts(cu_seqlens: torch.Tensor, T: int) -> torch.Tensor:
    """int32 [T]: index of the first token of each token's document; a token behind the last
    boundary is a document of its own."""
    cu = cu_seqlens.to(torch.int64).contiguous()
    pos = torch.arange(T, device=cu.device)
    seg = torch.searchsorted(cu, pos, right=True) - 1
    start = cu[seg.clamp_min(0)]
    inside = (seg >= 0) & (pos < cu[-1])
    return torch.where(inside, start, pos).to(torch.int32)


def causal_conv1d_reference(x, weight, bias, cu_seqlens, silu: bool):
    """Tensor-op form: K shifted copies of ``x`` masked at document starts."""
    T, C = x.shape
    K = weight.shape[1]
    start = document_starts(cu_seqlens, T).long()
    pos = torch.arange(T, device=x.device)
    acc = torch.zeros(T, C, dtype=torch.float32, device=x.device)
    xf = x.float()
    for j in range(K):
        shift = K - 1 - j
        src = pos - shift
        ok = (src >= start).unsqueeze(-1)
        acc = acc + torch.where(ok, xf[src.clamp_min(0)], torch.zeros((), device=x.device)) * weight[:, j].float()
    if bias is not None:
        acc = acc + bias.float()
    if silu:
        acc = F.silu(acc)
    return acc.to(x.dtype)


class _CausalConv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, doc_start, silu):
        global _launches
        T, C = x.shape
        K = weight.shape[1]
        if x.stride(1) != 1:
            x = x.contiguous()
        w = weight.to(torch.bfloat16).contiguous()
        b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        y = torch.empty((T, C), dtype=x.dtype, device=x.device)
        _lib.check(_lib.cuda_lib().xb_causal_conv1d_fwd(
            x.data_ptr(), x.stride(0), w.data_ptr(), _lib.ptr(b), doc_start.data_ptr(), y.data_ptr(),
            y.stride(0), T, C, K, int(silu), _lib.stream_ptr()), "xb_causal_conv1d_fwd")
        _launches += 1
        ctx.save_for_backward(x, w, b if b is not None else x.new_empty(0), doc_start)
        ctx.silu, ctx.has_bias = bool(silu), bias is not None
        ctx.w_dtype = weight.dtype
        ctx.b_dtype = None if bias is None else bias.dtype
        return y

    @staticmethod
    def backward(ctx, dy):
        global _launches
        x, w, b, doc_start = ctx.saved_tensors
        T, C = x.shape
        K = w.shape[1]
        lib = _lib.cuda_lib()
        if dy.stride(1) != 1 or dy.stride(0) % 8 or dy.data_ptr() % 16:
            dy = dy.contiguous()
        dpre = torch.empty((T, C), dtype=torch.bfloat16, device=x.device)
        dx = torch.empty((T, C), dtype=torch.bfloat16, device=x.device)
        chunks = lib.xb_causal_conv1d_bwd_chunks(T)
        partial = torch.empty((chunks, C, K + 1), dtype=torch.float32, device=x.device)
        _lib.check(lib.xb_causal_conv1d_bwd(
            dy.data_ptr(), dy.stride(0), x.data_ptr(), x.stride(0), w.data_ptr(),
            b.data_ptr() if ctx.has_bias else None, doc_start.data_ptr(), dpre.data_ptr(),
            dx.data_ptr(), dx.stride(0), partial.data_ptr(), T, C, K, int(ctx.silu),
            _lib.stream_ptr()), "xb_causal_conv1d_bwd")
        _launches += 3
        tot = partial.sum(0)
        dw = tot[:, :K].to(ctx.w_dtype)
        db = tot[:, K].to(ctx.b_dtype) if ctx.has_bias else None
        return dx, dw, db, None, None


def _kernel_ok(x: torch.Tensor, weight: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 8 == 0
            and x.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and weight.shape[1] <= MAX_TAPS)


def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                  cu_seqlens: torch.Tensor, silu: bool = True,
                  doc_start: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T, C], weight [C, K], bias [C] or None -> [T, C]."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and not _kernel_ok(x, weight):
        x = x.contiguous()
    if _kernel_ok(x, weight):
        if doc_start is None:
            doc_start = document_starts(cu_seqlens.to(x.device), x.shape[0])
        return _CausalConv1d.apply(x, weight, bias, doc_start, silu)
    return causal_conv1d_reference(x, weight, bias, cu_seqlens.to(x.device), silu)


def quant4_supported(w: torch.Tensor, fmt: str, group: int) -> bool:
    return (w.is_cuda and fmt in _FMT_CODE and w.dtype in (torch.bfloat16, torch.float32)
            and group in (16, 32, 64, 128) and w.numel() % group == 0 and w.numel() > 0)


def quant4(w: torch.Tensor, fmt: str, group: int) -> Dict[str, torch.Tensor]:
    """4-bit ``parts`` (the dictionary ``ops.quantize.quantize_weight`` returns) of a weight that lives
    on the GPU, by the quantiser kernel: the same codes and scales as the tensor-op definitions."""
    global _launches
    w = w.contiguous()
    n = w.numel()
    dev = w.device
    packed = torch.empty(n // 2, dtype=torch.uint8, device=dev)
    byte_scale = fmt in ("nvfp4", "mxfp4")
    scale = torch.empty(n // group, dtype=torch.uint8 if byte_scale else torch.float32, device=dev)
    gmax = gs = None
    if fmt == "nvfp4":
        gmax = w.abs().max().float().reshape(1)
        gs = torch.empty(1, dtype=torch.float32, device=dev)
    _lib.check(_lib.cuda_lib().xb_quant4(w.data_ptr(), int(w.dtype == torch.float32), _lib.ptr(gmax), packed.data_ptr(),
                                         scale.data_ptr(), _lib.ptr(gs), n, group, _FMT_CODE[fmt], _lib.stream_ptr()),
               "xb_quant4")
    _launches += 1
    parts = {"packed": packed, "scale": scale}
    if fmt == "nvfp4":
        parts["global_scale"] = gs
    return parts


def dequant4(parts: Dict[str, torch.Tensor], fmt: str, group: int, shape) -> torch.Tensor:
    """bf16 weight of ``shape`` from 4-bit ``parts`` (``packed``, ``scale`` and, for nvfp4,
    ``global_scale``) that live on the GPU."""
    global _launches
    n = 1
    for s in shape:
        n *= int(s)
    packed = parts["packed"].contiguous()
    scale = parts["scale"].contiguous()
    if fmt in ("nf4", "int4"):
        scale = scale.float()
    gs = parts["global_scale"].float().contiguous() if fmt == "nvfp4" else None
    if n % 8 or group % 8 or packed.data_ptr() % 4:
        raise ValueError(f"dequant4 needs element count and group size divisible by 8 (got {n}, {group})")
    out = torch.empty(n, dtype=torch.bfloat16, device=packed.device)
    _lib.check(_lib.cuda_lib().xb_dequant4(packed.data_ptr(), scale.data_ptr(), _lib.ptr(gs),
                                           out.data_ptr(), n, group, _FMT_CODE[fmt],
                                           _lib.stream_ptr()), "xb_dequant4")
    _launches += 1
    return out.reshape(*shape)
