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


def _pad_last(t: torch.Tensor, multiple: int = 128) -> torch.Tensor:
    pad = (-t.shape[-1]) % multiple
    return torch.nn.functional.pad(t, (0, pad)) if pad else t


class _QuantizedWeight:
    """e4m3 copies of one weight: ``[N, Kp]`` for the forward GEMM and ``[Kp, Np]`` (the transpose, the
    same 128 x 128 blocks) for the input-gradient GEMM; ``Kp`` / ``Np`` are the sizes padded to 128."""
    __slots__ = ("q_nk", "s_nk", "q_kn", "s_kn", "epoch", "ptr")


def quantized_weight(w: torch.Tensor, need_transpose: bool) -> _QuantizedWeight:
    """Quantised copies of ``w``, kept on the parameter object until the optimizers announce changed
    weights (``ops.fp8_grouped.invalidate_weight_cache``): with gradient accumulation and recomputation a
    weight is used many times per step and quantised once.  ``XORL_B200_FP8_WEIGHT_CACHE=0`` quantises
    on every use instead (no fp8 copy of the model stays resident)."""
    import os
    from ..ops import fp8_gemm, fp8_grouped
    use_cache = os.environ.get("XORL_B200_FP8_WEIGHT_CACHE", "1") == "1"
    c = getattr(w, "_xb_fp8_cache", None) if use_cache else None
    if c is None or c.epoch != fp8_grouped._weight_epoch or c.ptr != w.data_ptr():
        c = _QuantizedWeight()
        with torch.no_grad():
            wp = _pad_last(w.detach())
            if wp.shape[0] % 128:
                wp = torch.nn.functional.pad(wp, (0, 0, 0, (-wp.shape[0]) % 128))
            c.q_nk, c.s_nk = fp8_gemm.quantize_blocks(wp)
        c.q_kn = c.s_kn = None
        c.epoch, c.ptr = fp8_grouped._weight_epoch, w.data_ptr()
        if use_cache:
            try:
                w._xb_fp8_cache = c
            except AttributeError:
                pass
    if need_transpose and c.q_kn is None:
        # square blocks: the transposed weight has the transposed codes and the transposed scale grid
        c.q_kn, c.s_kn = c.q_nk.t().contiguous(), c.s_nk.t().contiguous()
    return c


class _FP8LinearFn(torch.autograd.Function):
    """y = x W^T on e4m3 operands (1 x 128 activation scales, 128 x 128 weight scales).  With
    ``fp8_backward`` the input gradient dx = dy W is an fp8 GEMM too (dy quantised along the output
    features); the weight gradient stays in the compute dtype (src/xorl/fp8_training/linear.py:85-333)."""

    @staticmethod
    def forward(ctx, x, w, fp8_backward: bool):
        from ..ops import fp8_gemm
        x2 = x.reshape(-1, x.shape[-1])
        N, K = w.shape
        qw = quantized_weight(w, need_transpose=False)
        aq, as_ = fp8_gemm.quantize_rows(_pad_last(x2))
        y = fp8_gemm.block_fp8_gemm(aq, as_, qw.q_nk, qw.s_nk, out_dtype=x.dtype)[:, :N]
        ctx.save_for_backward(x2, w)
        ctx.fp8_backward = fp8_backward
        ctx.x_shape = x.shape
        return y.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        N, K = w.shape
        dy2 = dy.reshape(-1, dy.shape[-1]).contiguous()
        from ..ops import fp8_gemm
        from ..ops.gemm import gemm
        on_kernel = dy2.is_cuda and dy2.dtype == torch.bfloat16
        dx = dw = None
        if ctx.needs_input_grad[0]:
            if ctx.fp8_backward:
                qw = quantized_weight(w, need_transpose=True)
                gq, gs = fp8_gemm.quantize_rows(_pad_last(dy2))
                dx = fp8_gemm.block_fp8_gemm(gq, gs, qw.q_kn, qw.s_kn, out_dtype=dy2.dtype)[:, :K]
            else:
                dx = gemm(dy2, w, b_mn=True) if on_kernel else dy2 @ w
            dx = dx.reshape(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            dw = gemm(dy2, x2, a_mn=True, b_mn=True, out_dtype=w.dtype) if on_kernel else dy2.t() @ x2
        return dx, dw, None


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


def _module_override(full: str, overrides) -> dict:
    """First pattern of ``train.fp8_training_module_overrides`` (globs on the full or the last name) that
    matches.  ``backward_mode`` (``fp8`` / ``bf16``) is the per-module choice that exists here; the block
    size is 128 everywhere, and amax margins, SmoothQuant and residual correction are not built."""
    import fnmatch
    short = full.rsplit(".", 1)[-1]
    for pattern, recipe in (overrides or {}).items():
        if fnmatch.fnmatch(full, pattern) or fnmatch.fnmatch(short, pattern):
            extra = {k: v for k, v in recipe.items()
                     if k != "backward_mode" and not (k == "block_size" and v == 128)
                     and not (k in ("activation_amax_scale", "weight_amax_scale") and v in (1, 1.0))
                     and not (k == "correction_mode" and v == "none") and not (k == "smoothquant_alpha" and not v)}
            if extra:
                raise NotImplementedError(f"fp8_training_module_overrides[{pattern!r}]: {sorted(extra)} cannot be "
                                          f"overridden per module (only backward_mode can)")
            if recipe.get("backward_mode", "fp8") not in ("fp8", "bf16"):
                raise ValueError(f"fp8_training_module_overrides[{pattern!r}].backward_mode must be fp8 or bf16")
            return dict(recipe)
    return {}


def inject_fp8_training(model: nn.Module, train_args) -> List[str]:
    validate_blackwell_policy(train_args)
    overrides = getattr(train_args, "fp8_training_module_overrides", None)
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
                mode = _module_override(full, overrides).get("backward_mode", train_args.fp8_training_backward)
                child.fp8_mode = "fp8" if mode == "fp8" else "bf16"
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
            mode = _module_override(full, overrides).get("backward_mode", train_args.fp8_training_backward)
            setattr(parent, cname, FP8Linear(child, mode == "fp8"))
            wrapped.append(full)
    return wrapped
