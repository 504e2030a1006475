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

    def _parts(self) -> Dict[str, torch.Tensor]:
        parts = {}
        for key, (pdt, pshape) in self.part_meta.items():
            raw = self.qparts[key].view(torch.uint8)
            n = math.prod(pshape) * torch.empty(0, dtype=pdt).element_size()
            parts[key] = raw[:n].view(pdt).reshape(pshape)
        return parts

    def quantisation_step(self) -> torch.Tensor:
        """Smallest spacing of the grid around each weight, ``[out, in]`` fp32: half the smallest code
        spacing times the element's scale (nf4: 0.5 * min code gap * absmax of its group; nvfp4 / mxfp4:
        0.5 * block scale (* tensor scale); int4: 0.5 * group scale; block fp8: the e4m3 unit spacing
        0.125 * block scale) (src/xorl/qlora/modules/{nf4,nvfp4,block_fp8}_linear.py ``_compute_aqn_step``)."""
        N, K = self.w_shape
        p = self._parts()
        if self.fmt == "block_fp8":
            s = p["scale"].float().reshape(-(-N // 128), -(-K // 128))
            return 0.125 * s.repeat_interleave(128, 0).repeat_interleave(128, 1)[:N, :K]
        if self.fmt == "nvfp4":
            s = p["scale"].view(torch.float8_e4m3fn).float().reshape(N, K // self.group) * p["global_scale"].float().reshape(())
            return 0.5 * s.repeat_interleave(self.group, 1)
        if self.fmt == "mxfp4":                                    # scales are stored as biased power-of-two exponents
            s = torch.exp2(p["scale"].float().reshape(N, K // self.group) - 127.0)
            return 0.5 * s.repeat_interleave(self.group, 1)
        s = p["scale"].float().reshape(N, K // self.group)
        if self.fmt == "nf4":
            gaps = (Q.NF4_VALUES[1:] - Q.NF4_VALUES[:-1]).min().item()
            return (0.5 * gaps) * s.repeat_interleave(self.group, 1)
        return 0.5 * s.repeat_interleave(self.group, 1)            # int4: unit code spacing

    def forward(self, x):
        w = self.dequantized_weight().to(x.dtype)
        if getattr(self, "enable_aqn", False) and self.training and torch.is_grad_enabled():
            # adaptive quantisation noise: Gaussian noise of the size of the grid spacing around each frozen
            # weight, fresh on every training forward (not in evaluation / reference passes), so the adapters
            # do not fit the rounding pattern of the base weights.  The step depends only on the stored
            # scales and is kept until the base weight is re-quantised.
            step = getattr(self, "_aqn_step", None)
            if step is None or step.device != w.device:
                step = self._aqn_step = self.quantisation_step().to(w.device, w.dtype)
            w = torch.addcmul(w, torch.randn_like(w), step, value=float(self.aqn_alpha))
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

    def quantize_parts(self, w: torch.Tensor) -> Dict[str, torch.Tensor]:
        """Packed storage (one raw-byte tensor per part, in the storage dtype) of a full-precision weight."""
        if tuple(w.shape) != tuple(self.w_shape):
            raise ValueError(f"expected a weight of shape {self.w_shape}, got {tuple(w.shape)}")
        return {k: _as_compute(t, self._store_dtype) for k, t in Q.quantize_weight(w.float(), self.fmt, self.group).items()}

    @torch.no_grad()
    def load_base_weight(self, w: torch.Tensor) -> None:
        """Quantise a full-precision weight into this module's packed storage."""
        for key, t in self.quantize_parts(w.cpu()).items():
            self.qparts[key].copy_(t.to(self.qparts[key].device))
        self._aqn_step = None


class PackedWeight(nn.Module):
    """Packed storage of one stacked expert tensor ``[E_local, K, N]``: the parts of the 4-bit / fp8
    codec as frozen raw-byte parameters (sharded and gathered by the ZeRO engine like any expert
    weight), dequantised to the compute dtype on use (src/xorl/qlora/modules/moe_experts.py)."""

    def __init__(self, shape, fmt: str, group: int, dtype, device, ep=None, std: float = 0.02):
        super().__init__()
        self.w_shape, self.fmt, self.group, self.ep = tuple(shape), fmt, group, ep
        self._store_dtype = dtype
        probe = Q.quantize_weight(torch.zeros(self.w_shape), fmt, group)
        self.part_meta = {k: (v.dtype, tuple(v.shape)) for k, v in probe.items()}
        self.qparts = nn.ParameterDict()
        es = torch.empty(0, dtype=dtype).element_size()
        for key, (pdt, pshape) in self.part_meta.items():
            nbytes = math.prod(pshape) * torch.empty(0, dtype=pdt).element_size()
            n = (nbytes + es - 1) // es
            p = nn.Parameter(torch.empty(n, dtype=dtype, device=device), requires_grad=False)
            p._xb_expert = True
            if ep is not None and ep[1] > 1:
                # every expert-parallel rank holds the bytes of its own experts: a 1-D tensor split evenly
                from ..parallel.ep import mark_ep
                mark_ep(p, ep[0], ep[1])
                p._xb_full_shape = (n * ep[1],)

            def mat(view_shape, dev, name, seed_, key=key):
                import zlib
                g = torch.Generator().manual_seed((seed_ * 1000003 + zlib.crc32(name.rsplit(".", 2)[0].encode())
                                                   + (ep[0] if ep else 0)) % (2 ** 63 - 1))
                w = torch.empty(self.w_shape).normal_(0.0, std, generator=g)
                return self.quantize_parts(w)[key].to(dev).reshape(view_shape)
            p._xb_materialize = mat
            self.qparts[key] = p

    def quantize_parts(self, w: torch.Tensor) -> Dict[str, torch.Tensor]:
        if tuple(w.shape) != self.w_shape:
            raise ValueError(f"expected experts of shape {self.w_shape}, got {tuple(w.shape)}")
        return {k: _as_compute(t, self._store_dtype) for k, t in Q.quantize_weight(w.float(), self.fmt, self.group).items()}

    def local_slice(self, full: torch.Tensor) -> torch.Tensor:
        """This rank's experts of a full ``[E, K, N]`` tensor."""
        if self.ep is None or self.ep[1] == 1 or full.shape[0] == self.w_shape[0]:
            return full
        El = self.w_shape[0]
        return full[self.ep[0] * El:(self.ep[0] + 1) * El]

    def dequantized(self) -> torch.Tensor:
        parts = {}
        for key, (pdt, pshape) in self.part_meta.items():
            raw = self.qparts[key].view(torch.uint8)
            n = math.prod(pshape) * torch.empty(0, dtype=pdt).element_size()
            parts[key] = raw[:n].view(pdt).reshape(pshape)
        cuda = self.qparts["packed"].is_cuda
        if cuda and self.fmt in ("nf4", "int4", "nvfp4", "mxfp4") and self.group % 8 == 0:
            from ..ops.seqmix import dequant4
            return dequant4(parts, self.fmt, self.group, self.w_shape)
        return Q.dequantize_weight(parts, self.fmt, self.group, self.w_shape, torch.bfloat16 if cuda else torch.float32)


_QUANTIZED_EXPERT_CLASSES: Dict[type, type] = {}


def quantize_experts_(experts: nn.Module, fmt: str, group: int) -> None:
    """Replaces the stacked ``gate_up_proj`` / ``down_proj`` parameters of an experts module by packed
    storage; the attributes keep working (they dequantise on access), so every expert path -- local,
    all-to-all, fused dispatch, LoRA -- runs unchanged on the frozen quantised base."""
    cls = type(experts)
    if cls not in _QUANTIZED_EXPERT_CLASSES:
        def prop(name):
            return property(lambda self: getattr(self, name + "_q").dequantized().to(self._q_compute_dtype))
        _QUANTIZED_EXPERT_CLASSES[cls] = type("Quantized" + cls.__name__, (cls,),
                                              {"gate_up_proj": prop("gate_up_proj"), "down_proj": prop("down_proj")})
    for name in ("gate_up_proj", "down_proj"):
        p = experts._parameters.pop(name)
        experts._q_compute_dtype = p.dtype
        experts.add_module(name + "_q", PackedWeight(tuple(getattr(p, "_xb_shape", p.shape)), fmt, group, p.dtype,
                                                     p.device, ep=getattr(p, "_xb_ep", None)))
    experts.__class__ = _QUANTIZED_EXPERT_CLASSES[cls]


def inject_qlora(model: nn.Module, lora_args) -> List[str]:
    from .target_manifest import resolve_targets, validate
    listed, manifest = resolve_targets(lora_args.lora_target_modules, getattr(lora_args, "lora_target_manifest", None))
    targets = tuple(listed or DEFAULT_TARGETS)
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
            q = QLoRALinear(child, lora_args.lora_rank, lora_args.lora_alpha, slices,
                            lora_args.quant_format, lora_args.quant_group_size,
                            lora_args.lora_b_init_std, lora_args.lora_b_init_seed)
            q.enable_aqn, q.aqn_alpha = bool(getattr(lora_args, "enable_aqn", False)), float(getattr(lora_args, "aqn_alpha", 1.0))
            setattr(parent, cname, q)
            wrapped.append(full)
    if True:
        # MoE experts: per-expert adapters (when the expert projections are targeted) over a packed base
        from ..models.moe import Experts
        from .lora import ExpertsLoRA
        for name, m in list(model.named_modules()):
            if isinstance(m, Experts) and not any(x in name for x in exclude) and "gate_up_proj" in m._parameters:
                proj = [p for p in ExpertsLoRA.PROJ if p in targets]
                if proj and getattr(m, "lora", None) is None and m.gate_up_proj.shape[2] == 2 * m.down_proj.shape[1]:
                    m.lora = ExpertsLoRA(m, lora_args.lora_rank, lora_args.lora_alpha, proj, lora_args.lora_b_init_std,
                                         hybrid_shared=bool(getattr(lora_args, "moe_hybrid_shared_lora", False)))
                quantize_experts_(m, lora_args.quant_format, lora_args.quant_group_size)
                wrapped.append(name)
    for n, p in model.named_parameters():
        p.requires_grad_(("lora_A" in n) or ("lora_B" in n))
    model._xb_lora_config = {"r": lora_args.lora_rank, "lora_alpha": lora_args.lora_alpha,
                             "target_modules": list(targets), "quant_format": lora_args.quant_format}
    if lora_args.lora_b_init_std:
        model._xb_lora_config.update(b_init_std=float(lora_args.lora_b_init_std), b_init_seed=int(lora_args.lora_b_init_seed or 0))
    if manifest is not None:
        validate(model, manifest)
    return wrapped
