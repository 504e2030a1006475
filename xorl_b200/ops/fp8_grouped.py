"""Block-scaled fp8 (e4m3) grouped expert GEMMs with power-of-two scales (``csrc/grouped_gemm_mx.cu``).

Scheme: activations carry one scale per row and 128-wide K block (1 x 128), stacked expert weights
one scale per 128 x 128 block -- the block shapes of the reference's ``block_fp8`` training
(src/xorl/fp8_training/grouped.py:116-330, src/xorl/ops/quantize/block_fp8_quantize.py:24-94).
Scales are powers of two stored as UE8M0 bytes (``2 ** (b - 127)``), the form the Blackwell tensor
core applies itself (``tcgen05.mma.kind::mxf8f6f4.block_scale``), so the grouped GEMM runs its whole
K loop on the tensor core without promoting partial sums through registers.  Rounding a scale up to
the next power of two costs at most one bit of the e4m3 range of a block.

``grouped_linear_fp8`` is the autograd function used by the expert MLP: forward and input gradient
in fp8 (or the input gradient in bf16 with ``backward="bf16"``), weight gradient in bf16 from the
saved bf16 activations.  The quantised weights of an expert tensor are cached until
``invalidate_weight_cache`` (called by the optimizers) says the weights changed.

Every function has a plain PyTorch restatement (``*_ref``) that is both the CPU lane and the test
oracle.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib
from .grad_sink import grad_target, mark_written

E4M3_MAX = 448.0
_launches = 0
_weight_epoch = 0


def launch_count() -> int:
    return _launches


def invalidate_weight_cache() -> None:
    """The weights changed (optimizer step, checkpoint load): cached quantised copies are stale."""
    global _weight_epoch
    _weight_epoch += 1


def sf_stride(k: int) -> int:
    """Row stride of a scale array for a reduction length ``k``: K / 128 rounded up to 16 bytes."""
    return (k // 128 + 15) // 16 * 16


# --------------------------------------------------------------------------------------------
# reference (CPU lane and oracle)
# --------------------------------------------------------------------------------------------
def pow2_scale_exponent(amax: torch.Tensor) -> torch.Tensor:
    """Smallest integer e with amax / 2**e <= 448 (0 where amax == 0), clamped to [-126, 126]."""
    r = amax.double() / E4M3_MAX
    m, ex = torch.frexp(r)
    e = torch.where(m == 0.5, ex - 1, ex)
    e = torch.where(amax > 0, e, torch.zeros_like(e))
    return e.clamp(-126, 126).to(torch.int32)


def _to_e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def quantize_rows_ref(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [M, K] -> (q float8_e4m3fn [M, K], exponent int32 [M, K/128])."""
    M, K = x.shape
    xb = x.float().view(M, K // 128, 128)
    e = pow2_scale_exponent(xb.abs().amax(-1))
    q = _to_e4m3(xb * torch.exp2(-e.float()).unsqueeze(-1)).view(M, K)
    return q, e


def quantize_weight_ref(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [E, K, N] -> (q float8_e4m3fn [E, K, N], exponent int32 [E, K/128, N/128])."""
    E, K, N = w.shape
    wb = w.float().view(E, K // 128, 128, N // 128, 128)
    e = pow2_scale_exponent(wb.abs().amax(dim=(2, 4)))
    q = _to_e4m3(wb * torch.exp2(-e.float())[:, :, None, :, None]).view(E, K, N)
    return q, e


def dequantize_rows_ref(q: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * torch.exp2(e.float()).unsqueeze(-1)).view(M, K)


def dequantize_weight_ref(q: torch.Tensor, e: torch.Tensor) -> torch.Tensor:
    E, K, N = q.shape
    return (q.float().view(E, K // 128, 128, N // 128, 128)
            * torch.exp2(e.float())[:, :, None, :, None]).view(E, K, N)


def grouped_rows_ref(x: torch.Tensor, w: torch.Tensor, seg: torch.Tensor) -> torch.Tensor:
    """Oracle of the fp8 grouped GEMM: quantise both operands, dequantise, multiply in fp32.
    x [R, K], w [E, K, N] -> [R, N] in x.dtype; rows outside every segment are zero."""
    xq, xe = quantize_rows_ref(x)
    wq, we = quantize_weight_ref(w)
    xd, wd = dequantize_rows_ref(xq, xe), dequantize_weight_ref(wq, we)
    out = x.new_zeros((x.shape[0], w.shape[2]))
    s = seg.tolist()
    for e in range(w.shape[0]):
        if s[e + 1] > s[e]:
            out[s[e]:s[e + 1]] = (xd[s[e]:s[e + 1]] @ wd[e]).to(x.dtype)
    return out


# --------------------------------------------------------------------------------------------
# CUDA path
# --------------------------------------------------------------------------------------------
def quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """bf16 [M, K] -> (q uint8 [M, K] holding e4m3 bits, scales uint8 [M, sf_stride(K)] UE8M0)."""
    global _launches
    assert x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 128 == 0
    if x.stride(1) != 1 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()
    M, K = x.shape
    q = torch.empty((M, K), device=x.device, dtype=torch.uint8)
    sf = torch.empty((M, sf_stride(K)), device=x.device, dtype=torch.uint8)
    _lib.check(_lib.cuda_lib().xb_quant_mx_rows(x.data_ptr(), x.stride(0), q.data_ptr(), q.stride(0),
                                                sf.data_ptr(), sf.stride(0), M, K, _lib.stream_ptr()),
               "xb_quant_mx_rows")
    _launches += 1
    return q, sf


class QuantizedExperts:
    """Both orientations of a stacked expert weight ``w [E, K, N]``:
    ``q_nk [E, N, K]`` + ``sf_nk [E, N/128, sf_stride(K)]`` (B operand of ``x @ w``) and
    ``q_kn [E, K, N]`` + ``sf_kn [E, K/128, sf_stride(N)]`` (B operand of ``dy @ w^T``)."""
    __slots__ = ("q_nk", "sf_nk", "q_kn", "sf_kn", "epoch", "ptr")


def quantize_experts(w: torch.Tensor) -> QuantizedExperts:
    global _launches
    assert w.is_cuda and w.dtype == torch.bfloat16 and w.dim() == 3
    E, K, N = w.shape
    assert K % 128 == 0 and N % 128 == 0, "expert weight dims must be multiples of 128 for block fp8"
    w = w.contiguous()
    qe = QuantizedExperts()
    dev = w.device
    qe.q_nk = torch.empty((E, N, K), device=dev, dtype=torch.uint8)
    qe.q_kn = torch.empty((E, K, N), device=dev, dtype=torch.uint8)
    qe.sf_nk = torch.full((E, N // 128, sf_stride(K)), 127, device=dev, dtype=torch.uint8)
    qe.sf_kn = torch.full((E, K // 128, sf_stride(N)), 127, device=dev, dtype=torch.uint8)
    _lib.check(_lib.cuda_lib().xb_quant_mx_weight(w.data_ptr(), qe.q_kn.data_ptr(), qe.sf_kn.data_ptr(),
                                                  qe.sf_kn.stride(1), qe.q_nk.data_ptr(), qe.sf_nk.data_ptr(),
                                                  qe.sf_nk.stride(1), E, K, N, _lib.stream_ptr()),
               "xb_quant_mx_weight")
    _launches += 3
    return qe


def cached_quantized_experts(w: torch.Tensor) -> QuantizedExperts:
    """Quantised copies of ``w``, reused while the weights have not changed.  The cache lives on the
    parameter object and is keyed by the storage address and the global weight epoch."""
    c = getattr(w, "_xb_mx_cache", None)
    if c is not None and c.epoch == _weight_epoch and c.ptr == w.data_ptr():
        return c
    qe = quantize_experts(w.detach())
    qe.epoch, qe.ptr = _weight_epoch, w.data_ptr()
    try:
        w._xb_mx_cache = qe
    except AttributeError:
        pass
    return qe


def grouped_rows_mx(xq: torch.Tensor, sfx: torch.Tensor, wq: torch.Tensor, sfw: torch.Tensor,
                    seg: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[rows of e] = dequant(xq)[rows of e] @ dequant(wq[e])^T with wq [E, N, K] (K contiguous)."""
    global _launches
    R, K = xq.shape
    E, N, K2 = wq.shape
    assert K == K2
    if out is None:
        out = torch.zeros((R, N), device=xq.device, dtype=torch.bfloat16)
    _lib.check(_lib.cuda_lib().xb_grouped_gemm_mx_rows(
        xq.data_ptr(), sfx.data_ptr(), wq.data_ptr(), sfw.data_ptr(), out.data_ptr(), seg.data_ptr(), E, R, N, K,
        xq.stride(0), out.stride(0), sfx.stride(0), sfw.stride(1), _lib.stream_ptr()), "xb_grouped_gemm_mx_rows")
    _launches += 1
    return out


class _GroupedLinearFP8(torch.autograd.Function):
    """y[rows of e] = x[rows of e] @ w[e], w [E, K, N], fp8 operands with block scales."""

    @staticmethod
    def forward(ctx, x, w, seg, backward_mode):
        from .moe import _grouped_wgrad_cuda  # noqa: F401  (bf16 weight gradient)
        qe = cached_quantized_experts(w)
        xq, sfx = quantize_rows(x)
        ctx.save_for_backward(x, seg)
        ctx.w, ctx.backward_mode = w, backward_mode
        return grouped_rows_mx(xq, sfx, qe.q_nk, qe.sf_nk, seg)

    @staticmethod
    def backward(ctx, dy):
        from .moe import _grouped_rows_cuda, _grouped_wgrad_cuda
        x, seg = ctx.saved_tensors
        w = ctx.w
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            if ctx.backward_mode == "fp8":
                qe = cached_quantized_experts(w)
                dq, sfd = quantize_rows(dy)
                dx = grouped_rows_mx(dq, sfd, qe.q_kn, qe.sf_kn, seg)      # dy @ w[e]^T
            else:
                dx = torch.zeros_like(x)
                _grouped_rows_cuda(dy, w, seg, dx, b_kmajor=True)
        dw = None
        if ctx.needs_input_grad[1]:
            tgt, fresh = grad_target(w)
            if tgt is not None:
                _grouped_wgrad_cuda(x, dy, seg, tgt, accumulate=not fresh)
                mark_written(w)
            else:
                dw = torch.empty_like(w)
                _grouped_wgrad_cuda(x, dy, seg, dw, accumulate=False)
        return dx, dw, None, None


def fp8_grouped_ok(x: torch.Tensor, w: torch.Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and w.dim() == 3
            and w.shape[1] % 128 == 0 and w.shape[2] % 128 == 0 and x.shape[0] % 128 == 0)


def grouped_linear_fp8(x: torch.Tensor, w: torch.Tensor, seg: torch.Tensor, backward: str = "fp8") -> torch.Tensor:
    """Grouped expert linear in block-scaled fp8.  CUDA: the tcgen05 block-scaled kernel.  CPU: the
    quantise / dequantise restatement with straight-through gradients (numerics of the same
    scheme, used by the CPU tests)."""
    if fp8_grouped_ok(x, w):
        return _GroupedLinearFP8.apply(x, w, seg, backward)
    if x.is_cuda:
        raise ValueError(f"block-fp8 experts need bf16 operands with 128-aligned shapes, got x {tuple(x.shape)} "
                         f"{x.dtype}, w {tuple(w.shape)} {w.dtype}")
    return _RefGroupedLinearFP8.apply(x, w, seg)


class _RefGroupedLinearFP8(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, seg):
        ctx.save_for_backward(x, w, seg)
        return grouped_rows_ref(x, w, seg)

    @staticmethod
    def backward(ctx, dy):
        x, w, seg = ctx.saved_tensors
        dx = grouped_rows_ref(dy, w.transpose(1, 2).contiguous(), seg)
        dw = torch.zeros_like(w)
        s = seg.tolist()
        for e in range(w.shape[0]):
            if s[e + 1] > s[e]:
                dw[e] = (x[s[e]:s[e + 1]].float().t() @ dy[s[e]:s[e + 1]].float()).to(w.dtype)
        return dx, dw, None
