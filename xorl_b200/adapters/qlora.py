"""QLoRA: frozen base weights stored quantised (nvfp4 / block_fp8 / nf4 / int4 / mxfp4), LoRA
adapters on top.  The packed bytes and their scales live in frozen parameters whose storage is
reinterpreted in the compute dtype, so the ZeRO engine shards and gathers them like any weight;
the forward dequantises to bf16 and runs the tcgen05 GEMM (src/xorl/qlora/modules/linear.py:29-369,
src/xorl/qlora/utils.py:68-346)."""
from __future__ import annotations

import math
from typing import Dict, List

import torch
from torch import nn

from ..models.layers import Linear
from ..ops import gemm as gemm_ops
from ..ops import quantize as Q
from .lora import DEFAULT_TARGETS, LoraLinear, _fused_slices


def _as_compute(t: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """Raw bytes of ``t`` viewed as ``dtype`` (padded to a whole element)."""
    b = t.contiguous().view(torch.uint8).reshape(-1)
    es = torch.empty(0, dtype=dtype).element_size()
    pad = (-b.numel()) % es
    if pad:
        b = torch.cat([b, b.new_zeros(pad)])
    return b.view(dtype)


class QLoRALinear(LoraLinear):
    def __init__(self, base: Linear, rank, alpha, slices, fmt: str, group: int, b_init_std=0.0, seed=0):
        super().__init__(base, rank, alpha, slices, b_init_std, seed)
        self.fmt, self.group = fmt, group
        shape = (base.out_features, base.in_features)
        self.w_shape = shape
        dt = base.weight.dtype if base.weight.dtype != torch.float32 else torch.float32
        probe = Q.quantize_weight(torch.zeros(shape), fmt, group)
        self.part_meta = {k: (v.dtype, tuple(v.shape)) for k, v in probe.items()}
        del self.weight
        std = 0.02

        def make(key):
            def mat(view_shape, device, name, seed_):
                # deferred quantisation: draw (or receive) the full-precision weight, quantise, keep
                # only the requested part as raw bytes
                import zlib
                g = torch.Generator().manual_seed((seed_ * 1000003 + zlib.crc32(name.rsplit(".", 1)[0].encode())) % (2 ** 63 - 1))
                w = torch.empty(shape).normal_(0.0, std, generator=g)
                part = Q.quantize_weight(w, fmt, group)[key]
                return _as_compute(part, self._store_dtype).to(device).reshape(view_shape)
            return mat

        self._store_dtype = dt
        self.qparts = nn.ParameterDict()
        for key, (pdt, pshape) in self.part_meta.items():
            nbytes = math.prod(pshape) * torch.empty(0, dtype=pdt).element_size()
            es = torch.empty(0, dtype=dt).element_size()
            p = nn.Parameter(torch.empty((nbytes + es - 1) // es, dtype=dt, device=base.weight.device),
                             requires_grad=False)
            p._xb_materialize = make(key)
            self.qparts[key] = p

    def dequantized_weight(self) -> torch.Tensor:
        parts = {}
        for key, (pdt, pshape) in self.part_meta.items():
            raw = self.qparts[key].view(torch.uint8)
            n = math.prod(pshape) * torch.empty(0, dtype=pdt).element_size()
            parts[key] = raw[:n].view(pdt).reshape(pshape)
        if self.qparts["packed"].is_cuda and self.fmt in ("nf4", "int4", "nvfp4", "mxfp4") \
                and self.group % 8 == 0 and math.prod(self.w_shape) % 8 == 0:
            from ..ops.seqmix import dequant4
            return dequant4(parts, self.fmt, self.group, self.w_shape)
        dt = torch.bfloat16 if self.qparts["packed"].is_cuda else torch.float32
        return Q.dequantize_weight(parts, self.fmt, self.group, self.w_shape, dt)

    def forward(self, x):
        w = self.dequantized_weight().to(x.dtype)
        y = gemm_ops.linear(x, w, self.bias)
        pieces, cur = [], 0
        for name, s, e in sorted(self.slices, key=lambda t: t[1]):
            d = gemm_ops.linear(gemm_ops.linear(x, self.lora_A[name]), self.lora_B[name]) * self.scaling
            if s > cur:
                pieces.append(y[..., cur:s])
            pieces.append(y[..., s:e] + d)
            cur = e
        if cur < self.out_features:
            pieces.append(y[..., cur:])
        return torch.cat(pieces, dim=-1) if len(pieces) > 1 else pieces[0]

    @torch.no_grad()
    def load_base_weight(self, w: torch.Tensor) -> None:
        """Quantise a full-precision weight into this module's packed storage."""
        parts = Q.quantize_weight(w.float().cpu(), self.fmt, self.group)
        for key, t in parts.items():
            self.qparts[key].copy_(_as_compute(t, self._store_dtype).to(self.qparts[key].device))


def inject_qlora(model: nn.Module, lora_args) -> List[str]:
    targets = tuple(lora_args.lora_target_modules or DEFAULT_TARGETS)
    exclude = tuple(lora_args.exclude_modules or ())
    wrapped = []
    for pname, parent in list(model.named_modules()):
        for cname, child in list(parent.named_children()):
            full = f"{pname}.{cname}" if pname else cname
            if not isinstance(child, Linear) or any(x in full for x in exclude) or cname == "lm_head":
                continue
            slices = _fused_slices(full, child, parent, targets)
            if not slices:
                continue
            setattr(parent, cname, QLoRALinear(child, lora_args.lora_rank, lora_args.lora_alpha, slices,
                                               lora_args.quant_format, lora_args.quant_group_size,
                                               lora_args.lora_b_init_std, lora_args.lora_b_init_seed))
            wrapped.append(full)
    for n, p in model.named_parameters():
        p.requires_grad_(("lora_A" in n) or ("lora_B" in n))
    model._xb_lora_config = {"r": lora_args.lora_rank, "lora_alpha": lora_args.lora_alpha,
                             "target_modules": list(targets), "quant_format": lora_args.quant_format}
    return wrapped
