"""RMSNorm (optionally fused with the residual add) — ``csrc/norm.cu`` on CUDA, torch on CPU.

Mirrors the behaviour of the reference RMSNorm module
(src/xorl/models/layers/normalization.py:628-799): ``y = x * rsqrt(mean(x^2) + eps) * w`` with an
optional pre-norm residual add that also returns the updated residual stream, and the
zero-centred ``(1 + w)`` variant.
"""
from __future__ import annotations

import torch

from . import _lib
from .grad_sink import deliver_param_grad

_launches = 0


def launch_count() -> int:
    return _launches


def _rmsnorm_ref(x, w, eps, zero_centered):
    xf = x.float()
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    wf = w.float() + 1.0 if zero_centered else w.float()
    return (xf * rstd * wf).to(x.dtype)


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, residual, w, eps, zero_centered):
        global _launches
        shape = x.shape
        H = shape[-1]
        x2 = x.reshape(-1, H)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        T = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(T, device=x.device, dtype=torch.float32)
        res2 = res_out = None
        if residual is not None:
            res2 = residual.reshape(-1, H)
            if not res2.is_contiguous():
                res2 = res2.contiguous()
            res_out = torch.empty_like(x2)
        lib = _lib.cuda_lib()
        _lib.check(lib.xb_rmsnorm_fwd(x2.data_ptr(), _lib.ptr(res2), w.data_ptr(), y.data_ptr(),
                                      _lib.ptr(res_out), rstd.data_ptr(), T, H, float(eps),
                                      int(zero_centered), _lib.stream_ptr()), "xb_rmsnorm_fwd")
        _launches += 1
        h = res_out if residual is not None else x2
        ctx.save_for_backward(h, rstd)
        ctx.w = w
        ctx.zero_centered = zero_centered
        ctx.shape = shape
        ctx.has_res = residual is not None
        if residual is not None:
            return y.reshape(shape), res_out.reshape(shape)
        return y.reshape(shape), None

    @staticmethod
    def backward(ctx, dy, dh):
        global _launches
        h, rstd = ctx.saved_tensors
        w = ctx.w
        T, H = h.shape
        dy2 = dy.reshape(T, H)
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dres = None
        if ctx.has_res and dh is not None:
            dres = dh.reshape(T, H)
            if not dres.is_contiguous():
                dres = dres.contiguous()
        lib = _lib.cuda_lib()
        rows = lib.xb_rmsnorm_bwd_partial_rows(T)
        partial = torch.empty(rows * H, device=h.device, dtype=torch.float32)
        dx = torch.empty_like(h)
        dw = torch.empty(H, device=h.device, dtype=torch.float32)
        _lib.check(lib.xb_rmsnorm_bwd(dy2.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(),
                                      _lib.ptr(dres), dx.data_ptr(), partial.data_ptr(), None,
                                      dw.data_ptr(), 0, T, H, int(ctx.zero_centered),
                                      _lib.stream_ptr()), "xb_rmsnorm_bwd")
        _launches += 2
        dx = dx.reshape(ctx.shape)
        dwg = deliver_param_grad(w, dw) if ctx.needs_input_grad[2] else None
        return dx, (dx if ctx.has_res else None), dwg, None, None


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6,
            residual: torch.Tensor | None = None, zero_centered: bool = False):
    """Returns ``y`` or, when ``residual`` is given, ``(y, x + residual)``."""
    if not x.is_cuda:
        if residual is not None:
            h = x + residual
            return _rmsnorm_ref(h, w, eps, zero_centered), h
        return _rmsnorm_ref(x, w, eps, zero_centered)
    if x.dtype != torch.bfloat16 or x.shape[-1] % 8 or x.shape[-1] > 16384:
        if residual is not None:
            h = x + residual
            return _rmsnorm_ref(h, w, eps, zero_centered), h
        return _rmsnorm_ref(x, w, eps, zero_centered)
    y, h = _RMSNorm.apply(x, residual, w, eps, zero_centered)
    if residual is not None:
        return y, h
    return y
