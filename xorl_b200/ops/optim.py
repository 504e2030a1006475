"""Optimizer kernels on flat fp32 buffers (``csrc/optim.cu``) with torch fallbacks for CPU."""
from __future__ import annotations

import math

import torch

from . import _lib

_launches = 0


def launch_count() -> int:
    return _launches


def adamw_step_(p, m, v, g, bf16_out, *, lr, beta1, beta2, eps, weight_decay, step,
                grad_scale: float = 1.0, clip_coef: torch.Tensor | None = None) -> None:
    """In-place AdamW on flat fp32 tensors; optionally writes the bf16 copy of the new weights.
    ``clip_coef`` is a 1-element device tensor multiplied into the gradient (no host sync)."""
    global _launches
    if p.is_cuda:
        assert p.dtype == m.dtype == v.dtype == g.dtype == torch.float32
        _lib.check(_lib.cuda_lib().xb_adamw(p.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(),
                                            _lib.ptr(bf16_out), p.numel(), float(lr), float(beta1),
                                            float(beta2), float(eps), float(weight_decay), int(step),
                                            float(grad_scale), _lib.ptr(clip_coef),
                                            _lib.stream_ptr()), "xb_adamw")
        _launches += 1
        return
    gg = g.float() * grad_scale
    if clip_coef is not None:
        gg = gg * clip_coef.float()
    p.mul_(1.0 - lr * weight_decay)
    m.mul_(beta1).add_(gg, alpha=1.0 - beta1)
    v.mul_(beta2).addcmul_(gg, gg, value=1.0 - beta2)
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    denom = (v.sqrt() / math.sqrt(bc2)).add_(eps)
    p.addcdiv_(m, denom, value=-lr / bc1)
    if bf16_out is not None:
        bf16_out.copy_(p)


def sumsq_(g: torch.Tensor, total: torch.Tensor, accumulate: bool) -> None:
    """total[0] (+)= ||g||^2 (fp32), no host sync."""
    global _launches
    if g.is_cuda and g.dtype == torch.float32:
        lib = _lib.cuda_lib()
        partial = torch.empty(lib.xb_sumsq_partial_count(), device=g.device, dtype=torch.float32)
        _lib.check(lib.xb_sumsq(g.data_ptr(), g.numel(), partial.data_ptr(), total.data_ptr(),
                                int(accumulate), _lib.stream_ptr()), "xb_sumsq")
        _launches += 2
        return
    s = g.float().pow(2).sum()
    if accumulate:
        total.add_(s)
    else:
        total.fill_(s)


def clip_coef_(sumsq: torch.Tensor, max_norm: float, norm_out: torch.Tensor,
               coef_out: torch.Tensor) -> None:
    global _launches
    if sumsq.is_cuda:
        _lib.check(_lib.cuda_lib().xb_clip_coef(sumsq.data_ptr(), float(max_norm),
                                                norm_out.data_ptr(), coef_out.data_ptr(),
                                                _lib.stream_ptr()), "xb_clip_coef")
        _launches += 1
        return
    norm = sumsq.sqrt()
    norm_out.copy_(norm)
    if max_norm > 0:
        coef_out.copy_(torch.clamp(max_norm / (norm + 1e-6), max=1.0))
    else:
        coef_out.fill_(1.0)


def cast_accum_(src_bf16: torch.Tensor, dst_f32: torch.Tensor, scale: float = 1.0,
                accumulate: bool = True) -> None:
    global _launches
    if src_bf16.is_cuda and src_bf16.dtype == torch.bfloat16 and dst_f32.dtype == torch.float32:
        _lib.check(_lib.cuda_lib().xb_cast_accum(src_bf16.data_ptr(), dst_f32.data_ptr(),
                                                 src_bf16.numel(), float(scale), int(accumulate),
                                                 _lib.stream_ptr()), "xb_cast_accum")
        _launches += 1
        return
    if accumulate:
        dst_f32.add_(src_bf16.to(dst_f32.dtype), alpha=scale)
    else:
        dst_f32.copy_(src_bf16.to(dst_f32.dtype) * scale)


def signsgd_step_(p, g, bf16_out, *, lr, weight_decay) -> None:
    global _launches
    if p.is_cuda:
        _lib.check(_lib.cuda_lib().xb_signsgd(p.data_ptr(), g.data_ptr(), _lib.ptr(bf16_out),
                                              p.numel(), float(lr), float(weight_decay),
                                              _lib.stream_ptr()), "xb_signsgd")
        _launches += 1
        return
    p.mul_(1.0 - lr * weight_decay).add_(torch.sign(g), alpha=-lr)
    if bf16_out is not None:
        bf16_out.copy_(p)


def stochastic_round_bf16(x: torch.Tensor, seed: int) -> torch.Tensor:
    """fp32 -> bf16 with stochastic rounding (src/xorl/optim/stochastic_round.py:22)."""
    global _launches
    out = torch.empty(x.shape, device=x.device, dtype=torch.bfloat16)
    if x.is_cuda:
        xc = x.contiguous()
        _lib.check(_lib.cuda_lib().xb_stochastic_round(xc.data_ptr(), out.data_ptr(), xc.numel(),
                                                       seed & 0xFFFFFFFF, _lib.stream_ptr()),
                   "xb_stochastic_round")
        _launches += 1
        return out
    g = torch.Generator().manual_seed(seed)
    bits = x.contiguous().view(torch.int32)
    r = torch.randint(0, 1 << 16, bits.shape, generator=g, dtype=torch.int32)
    rounded = ((bits + r) & ~0xFFFF)
    return rounded.view(torch.float32).to(torch.bfloat16)
