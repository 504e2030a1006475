"""SwiGLU: ``silu(gate) * up`` on a fused ``[T, 2I]`` activation (``csrc/elementwise.cu``).

Matches src/xorl/ops/fused_silu_and_mul.py:23-359 of the reference, including the option to round
``silu(gate)`` to bf16 before the multiply."""
from __future__ import annotations

import torch

from . import _lib

_launches = 0


def launch_count() -> int:
    return _launches


def swiglu_reference(gu: torch.Tensor, two_round: bool = True) -> torch.Tensor:
    I = gu.shape[-1] // 2
    g, u = gu[..., :I], gu[..., I:]
    s = torch.nn.functional.silu(g.float())
    if two_round and gu.dtype != torch.float32:
        s = s.to(gu.dtype).float()
    return (s * u.float()).to(gu.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu, two_round):
        global _launches
        shape = gu.shape
        gu2 = gu.reshape(-1, shape[-1])
        if not gu2.is_contiguous():
            gu2 = gu2.contiguous()
        T, I2 = gu2.shape
        out = torch.empty((T, I2 // 2), device=gu.device, dtype=gu.dtype)
        _lib.check(_lib.cuda_lib().xb_swiglu_fwd(gu2.data_ptr(), out.data_ptr(), T, I2 // 2,
                                                 int(two_round), _lib.stream_ptr()), "xb_swiglu_fwd")
        _launches += 1
        ctx.save_for_backward(gu2)
        ctx.shape = shape
        return out.reshape(*shape[:-1], I2 // 2)

    @staticmethod
    def backward(ctx, dout):
        global _launches
        (gu2,) = ctx.saved_tensors
        T, I2 = gu2.shape
        d2 = dout.reshape(T, I2 // 2)
        if not d2.is_contiguous():
            d2 = d2.contiguous()
        dgu = torch.empty_like(gu2)
        _lib.check(_lib.cuda_lib().xb_swiglu_bwd(d2.data_ptr(), gu2.data_ptr(), dgu.data_ptr(), T,
                                                 I2 // 2, _lib.stream_ptr()), "xb_swiglu_bwd")
        _launches += 1
        return dgu.reshape(ctx.shape), None


def swiglu(gu: torch.Tensor, two_round: bool = True) -> torch.Tensor:
    if gu.is_cuda and gu.dtype == torch.bfloat16 and (gu.shape[-1] // 2) % 8 == 0:
        return _SwiGLU.apply(gu, two_round)
    return swiglu_reference(gu, two_round)
