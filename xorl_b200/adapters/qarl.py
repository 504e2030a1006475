"""Quantisation-aware RL: fake-quant (NVFP4 / FP8, straight-through) on linear weights so the
policy being trained sees the numerics of the quantised weights it is synced as
(src/xorl/qarl/fake_quant.py)."""
from __future__ import annotations

from typing import List

import torch
from torch import nn

from ..models.layers import Linear
from ..ops import gemm as gemm_ops
from ..ops import quantize as Q


def fake_quant(w: torch.Tensor, fmt: str) -> torch.Tensor:
    """Quantise-dequantise with a straight-through gradient."""
    with torch.no_grad():
        if fmt == "nvfp4":
            K = w.shape[-1]
            pad = (-K) % 16
            wp = torch.nn.functional.pad(w, (0, pad)) if pad else w
            p, s, g = Q.nvfp4_quantize(wp, 16)
            dq = Q.nvfp4_dequantize(p, s, g, wp.shape, 16, w.dtype)[..., :K]
        elif fmt == "fp8":
            q, s = Q.block_fp8_quantize_128x128(w)
            dq = Q.block_fp8_dequantize_128x128(q, s, 128, w.dtype)
        else:
            dq = w
    return w + (dq - w).detach()


class FakeQuantLinear(nn.Module):
    def __init__(self, base: Linear, fmt: str):
        super().__init__()
        self.in_features, self.out_features = base.in_features, base.out_features
        self.weight, self.bias, self.fmt = base.weight, base.bias, fmt

    def forward(self, x):
        return gemm_ops.linear(x, fake_quant(self.weight, self.fmt), self.bias)


def inject_fake_quant(model: nn.Module, train_args) -> List[str]:
    fmt = train_args.qarl_sync_format
    targets = train_args.qarl_target_modules
    exclude = tuple(train_args.qarl_exclude_modules or ()) + ("lm_head",)
    wrapped = []
    for pname, parent in list(model.named_modules()):
        for cname, child in list(parent.named_children()):
            full = f"{pname}.{cname}" if pname else cname
            if isinstance(child, Linear) and not any(x in full for x in exclude) and \
                    (not targets or any(t in full for t in targets)):
                setattr(parent, cname, FakeQuantLinear(child, fmt))
                wrapped.append(full)
    return wrapped
