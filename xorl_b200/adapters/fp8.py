"""Block-fp8 training: linears whose forward (and optionally backward) GEMMs run on e4m3 operands
with 1x128 activation scales and 128x128 (or row-wise 1x128) weight scales, master weights stay
bf16/fp32 (src/xorl/fp8_training/linear.py:85-333, grouped.py, utils.py:81).  On sm_100a the GEMM is
``csrc/quant.cu`` (tcgen05 ``kind::f8f6f4`` with per-K-block scale promotion); elsewhere the
quantise -> dequantise -> matmul reference keeps the numerics identical up to accumulation order.
The reference refuses fp8 training on Blackwell unless ``fp8_training_allow_blackwell`` is set
(src/xorl/fp8_training/config_compat.py:293-306); the same key is honoured here."""
from __future__ import annotations

from typing import List

import torch
from torch import nn

from ..models.layers import Linear
from ..ops import quantize as Q


class _FP8LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, fp8_backward: bool):
        x2 = x.reshape(-1, x.shape[-1])
        K = x2.shape[1]
        pad = (-K) % 128
        if pad:
            x2p = torch.nn.functional.pad(x2, (0, pad))
            wp = torch.nn.functional.pad(w, (0, pad))
        else:
            x2p, wp = x2, w
        from ..ops import fp8_gemm
        aq, as_ = fp8_gemm.quantize_rows(x2p)
        bq, bs = fp8_gemm.quantize_blocks(wp)
        y = fp8_gemm.block_fp8_gemm(aq, as_, bq, bs, out_dtype=x.dtype)
        ctx.save_for_backward(x2, w)
        ctx.fp8_backward = fp8_backward
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        from ..ops.gemm import gemm
        if dy2.is_cuda and dy2.dtype == torch.bfloat16:
            dx = gemm(dy2.contiguous(), w, b_mn=True)
            dw = gemm(dy2.contiguous(), x2, a_mn=True, b_mn=True, out_dtype=w.dtype)
        else:
            dx = dy2 @ w
            dw = dy2.t() @ x2
        return dx.reshape(ctx.x_shape), dw, None


class FP8Linear(nn.Module):
    def __init__(self, base: Linear, fp8_backward: bool = True):
        super().__init__()
        self.in_features, self.out_features = base.in_features, base.out_features
        self.weight, self.bias = base.weight, base.bias
        self.fp8_backward = fp8_backward

    def forward(self, x):
        y = _FP8LinearFn.apply(x, self.weight, self.fp8_backward)
        return y if self.bias is None else y + self.bias


def validate_blackwell_policy(train_args) -> None:
    cap = torch.cuda.get_device_capability()[0] if torch.cuda.is_available() else 0
    if cap >= 10 and not train_args.fp8_training_allow_blackwell:
        raise ValueError("fp8 training on Blackwell needs train.fp8_training_allow_blackwell=true "
                         "(validated numerics artifact)")


def inject_fp8_training(model: nn.Module, train_args) -> List[str]:
    validate_blackwell_policy(train_args)
    targets = train_args.fp8_training_target_modules
    exclude = tuple(train_args.fp8_training_exclude_modules or ()) + ("lm_head",)
    n_layers = getattr(model.config, "num_hidden_layers", 0)
    skip_first, skip_last = train_args.fp8_training_num_first_layers_bf16, train_args.fp8_training_num_last_layers_bf16
    wrapped = []
    from ..models.moe import Experts

    def layer_skipped(full: str) -> bool:
        parts = full.split(".")
        if "layers" in parts:
            li = int(parts[parts.index("layers") + 1])
            return li < skip_first or li >= n_layers - skip_last
        return False

    for pname, parent in list(model.named_modules()):
        for cname, child in list(parent.named_children()):
            full = f"{pname}.{cname}" if pname else cname
            if isinstance(child, Experts):
                # stacked routed experts: both grouped GEMMs of the expert MLP run in block-scaled fp8
                # (1 x 128 activation scales, 128 x 128 weight scales; ops/fp8_grouped.py)
                if any(x in full for x in exclude) or (targets and not any(t in full for t in targets)) \
                        or layer_skipped(full):
                    continue
                child.fp8_mode = "fp8" if train_args.fp8_training_backward == "fp8" else "bf16"
                wrapped.append(full)
                continue
            if not isinstance(child, Linear) or any(x in full for x in exclude):
                continue
            if targets and not any(t in full for t in targets):
                continue
            parts = full.split(".")
            if "layers" in parts:
                li = int(parts[parts.index("layers") + 1])
                if li < skip_first or li >= n_layers - skip_last:
                    continue
            setattr(parent, cname, FP8Linear(child, train_args.fp8_training_backward == "fp8"))
            wrapped.append(full)
    return wrapped
