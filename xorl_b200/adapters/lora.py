"""LoRA: low-rank adapters on linear layers, fused-projection aware, with PEFT-format export.

``inject_lora`` wraps every targeted ``Linear`` so that ``y = x W^T + (alpha/r) (x A^T) B^T`` with the
base weight frozen; only ``lora_A`` / ``lora_B`` are trainable and checkpointed.  Targets are given
by HF-style names (``q_proj``, ``v_proj``, ``gate_proj`` ...): a name that is part of a fused
projection (``qkv_proj``, ``gate_up_proj``) becomes a *delta* adapter restricted to that slice of
the fused output, which is numerically the adapter of the unfused module
(src/xorl/lora/modules/linear.py:23-273, src/xorl/lora/utils.py:465,1109).  ``merge_lora`` folds the
update into the base weight (ReLoRA-style merges every ``merge_lora_interval`` steps).
"""
from __future__ import annotations

import json
import math
import os
from contextlib import contextmanager
from typing import Dict, Iterable, List, Optional, Tuple

import torch
from torch import nn

from ..models.layers import Linear
from ..ops import gemm as gemm_ops

FUSED_PARTS = {"qkv_proj": ("q_proj", "k_proj", "v_proj"), "gate_up_proj": ("gate_proj", "up_proj")}
DEFAULT_TARGETS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")


class LoraLinear(nn.Module):
    """A frozen base ``Linear`` plus one low-rank adapter per output slice."""

    def __init__(self, base: Linear, rank: int, alpha: float, slices: List[Tuple[str, int, int]],
                 b_init_std: float = 0.0, seed: int = 0):
        super().__init__()
        self.in_features, self.out_features = base.in_features, base.out_features
        self.weight = base.weight
        self.bias = base.bias
        self.weight.requires_grad_(False)
        if self.bias is not None:
            self.bias.requires_grad_(False)
        self.rank, self.scaling = rank, alpha / rank
        self.slices = slices                      # (hf name, start row, end row) of the fused output
        dt, dev = base.weight.dtype, base.weight.device
        self.lora_A = nn.ParameterDict()
        self.lora_B = nn.ParameterDict()
        for name, s, e in slices:
            a = torch.empty(rank, self.in_features, dtype=dt, device=dev)
            b = torch.empty(e - s, rank, dtype=dt, device=dev)
            self.lora_A[name] = nn.Parameter(a)
            self.lora_B[name] = nn.Parameter(b)
            self.lora_A[name]._xb_lora = "A"
            self.lora_B[name]._xb_lora = "B" if b_init_std == 0.0 else "B_random"
        self.b_init_std = b_init_std

    def forward(self, x):
        y = gemm_ops.linear(x, self.weight, self.bias)
        if not getattr(self, "enabled", True):
            return y                              # reference pass: the frozen base model alone
        full = len(self.slices) == 1 and self.slices[0][1] == 0 and self.slices[0][2] == self.out_features
        deltas = []
        for name, s, e in self.slices:
            d = gemm_ops.linear(gemm_ops.linear(x, self.lora_A[name]), self.lora_B[name]) * self.scaling
            if full:
                return y + d
            deltas.append((s, e, d))
        pieces, cur = [], 0
        for s, e, d in sorted(deltas, key=lambda t: t[0]):
            if s > cur:
                pieces.append(y[..., cur:s])
            pieces.append(y[..., s:e] + d)
            cur = e
        if cur < self.out_features:
            pieces.append(y[..., cur:])
        return torch.cat(pieces, dim=-1)

    @torch.no_grad()
    def merge(self) -> None:
        for name, s, e in self.slices:
            delta = (self.lora_B[name].float() @ self.lora_A[name].float()) * self.scaling
            self.weight[s:e] += delta.to(self.weight.dtype)
            self.lora_B[name].zero_()


class ExpertsLoRA(nn.Module):
    """Per-expert low-rank adapters on the stacked expert weights of a MoE block: for every targeted
    projection ``p`` in gate_proj / up_proj / down_proj two trainable tensors ``p_lora_A [E, in, r]``
    and ``p_lora_B [E, r, out]`` (names and shapes of src/xorl/models/layers/moe/lora.py:13-15), the
    base expert weights frozen.  Lives as ``experts.lora``; the expert MLP adds
    ``(alpha / r) (x A_e) B_e`` with two extra grouped GEMMs per projection.  Under expert
    parallelism the adapter tensors hold the local experts and are sharded like the expert weights.

    ``hybrid_shared`` (``lora.moe_hybrid_shared_lora``): the factor on the hidden-size side is one matrix for
    all experts -- gate / up ``A [1, H, r]`` with per-expert ``B``, down ``B [1, r, H]`` with per-expert
    ``A`` (src/xorl/models/layers/moe/lora.py:206-236).  A shared factor is an ordinary replicated
    parameter (sharded and reduced with the dense ones, also across expert-parallel ranks) and its product
    is one dense GEMM over all rows instead of a grouped one."""
    PROJ = ("gate_proj", "up_proj", "down_proj")

    def __init__(self, experts, rank: int, alpha: float, targets: Iterable[str], b_init_std: float = 0.0,
                 hybrid_shared: bool = False):
        super().__init__()
        E, H, I2 = experts.gate_up_proj.shape
        I = experts.down_proj.shape[1]
        if I2 != 2 * I:
            raise NotImplementedError("expert LoRA needs gated experts (gate_up_proj of width 2 I)")
        dims = {"gate_proj": (H, I), "up_proj": (H, I), "down_proj": (I, H)}
        self.rank, self.scaling = rank, alpha / rank
        self.targets = tuple(p for p in self.PROJ if p in targets)
        dt, dev = experts.gate_up_proj.dtype, experts.gate_up_proj.device
        ep = getattr(experts.gate_up_proj, "_xb_ep", None)
        self.hybrid_shared = bool(hybrid_shared)
        for p in self.targets:
            fin, fout = dims[p]
            ea = 1 if hybrid_shared and p != "down_proj" else E
            eb = 1 if hybrid_shared and p == "down_proj" else E
            A = nn.Parameter(torch.empty(ea, fin, rank, dtype=dt, device=dev))
            B = nn.Parameter(torch.empty(eb, rank, fout, dtype=dt, device=dev))
            A._xb_lora, B._xb_lora = "A", ("B" if b_init_std == 0.0 else "B_random")
            for t, n in ((A, ea), (B, eb)):
                if n == 1 and hybrid_shared:
                    continue                                   # shared over the experts: a replicated dense parameter
                t._xb_expert = True
                if ep is not None:
                    from ..parallel.ep import mark_ep
                    mark_ep(t, ep[0], ep[1])
            setattr(self, f"{p}_lora_A", A)
            setattr(self, f"{p}_lora_B", B)
        for w in (experts.gate_up_proj, experts.down_proj, experts.gate_up_bias, experts.down_bias):
            if w is not None:
                w.requires_grad_(False)

    def tensors(self) -> Optional[dict]:
        if not getattr(self, "enabled", True):
            return None                           # reference pass: the frozen base experts alone
        out = {"scaling": self.scaling}
        for p in self.targets:
            out[p] = (getattr(self, f"{p}_lora_A"), getattr(self, f"{p}_lora_B"))
        return out

    @torch.no_grad()
    def merge_into(self, experts) -> None:
        """W += scaling * A B per expert, then B restarts at zero."""
        I = experts.down_proj.shape[1]
        for p in self.targets:
            A, B = getattr(self, f"{p}_lora_A"), getattr(self, f"{p}_lora_B")
            E = max(A.shape[0], B.shape[0])
            delta = torch.bmm(A.float().expand(E, -1, -1), B.float().expand(E, -1, -1)) * self.scaling
            if p == "gate_proj":
                experts.gate_up_proj[:, :, :I] += delta.to(experts.gate_up_proj.dtype)
            elif p == "up_proj":
                experts.gate_up_proj[:, :, I:] += delta.to(experts.gate_up_proj.dtype)
            else:
                experts.down_proj += delta.to(experts.down_proj.dtype)
            B.zero_()


def _fused_slices(module_name: str, linear: Linear, parent, targets: Iterable[str]):
    leaf = module_name.rsplit(".", 1)[-1]
    if leaf in FUSED_PARTS:
        parts = FUSED_PARTS[leaf]
        if leaf == "qkv_proj":
            sizes = [parent.Hq * parent.D, parent.Hkv * parent.D, parent.Hkv * parent.D]
        else:
            sizes = [linear.out_features // 2] * 2
        out, off = [], 0
        for p, n in zip(parts, sizes):
            if p in targets:
                out.append((p, off, off + n))
            off += n
        return out
    if leaf in targets:
        return [(leaf, 0, linear.out_features)]
    return []


def inject_lora(model: nn.Module, lora_args) -> List[str]:
    """Replaces targeted linears by ``LoraLinear`` and freezes everything else.  Returns the names
    of the wrapped modules."""
    from .target_manifest import resolve_targets, validate
    listed, manifest = resolve_targets(lora_args.lora_target_modules, getattr(lora_args, "lora_target_manifest", None))
    targets = tuple(listed or DEFAULT_TARGETS)
    if "all-linear" in targets:
        targets = DEFAULT_TARGETS
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
            setattr(parent, cname, LoraLinear(child, lora_args.lora_rank, lora_args.lora_alpha, slices,
                                              lora_args.lora_b_init_std, lora_args.lora_b_init_seed))
            wrapped.append(full)
    # stacked routed experts of MoE blocks (src/xorl/lora/utils.py:1618 inject_lora_into_model_with_moe)
    from ..models.moe import Experts
    for name, mod in list(model.named_modules()):
        if isinstance(mod, Experts) and not any(x in name for x in exclude) \
                and any(p in targets for p in ExpertsLoRA.PROJ) and getattr(mod, "activation", None) is None:
            mod.lora = ExpertsLoRA(mod, lora_args.lora_rank, lora_args.lora_alpha, targets, lora_args.lora_b_init_std,
                                   hybrid_shared=bool(getattr(lora_args, "moe_hybrid_shared_lora", False)))
            wrapped.append(name)
    for n, p in model.named_parameters():
        p.requires_grad_(("lora_A" in n) or ("lora_B" in n))
    model._xb_lora_config = {"r": lora_args.lora_rank, "lora_alpha": lora_args.lora_alpha,
                             "target_modules": list(targets)}
    if getattr(lora_args, "moe_hybrid_shared_lora", False):
        model._xb_lora_config["moe_hybrid_shared_lora"] = True
    if lora_args.lora_b_init_std:
        model._xb_lora_config.update(b_init_std=float(lora_args.lora_b_init_std), b_init_seed=int(lora_args.lora_b_init_seed or 0))
    if manifest is not None:
        validate(model, manifest)                   # exact adapter coverage, before any sharding or step
    return wrapped


def init_lora_parameter_(name: str, p: torch.Tensor, rank: int, seed: int = 0, b_std: float = 0.0) -> None:
    """Kaiming-uniform A (as PEFT), zero (or N(0, b_std)) B."""
    import zlib
    g = torch.Generator().manual_seed((seed * 1000003 + zlib.crc32(name.encode())) % (2 ** 63 - 1))
    if name.endswith("_lora_A"):
        # stacked expert adapters [E, in, r]: the same uniform bound per expert, fan-in = in
        bound = 1.0 / math.sqrt(p.shape[-2])
        p.copy_(((torch.rand(p.shape, generator=g) * 2 - 1) * bound * math.sqrt(3.0)).to(p.device))
    elif ".lora_A." in name:
        bound = 1.0 / math.sqrt(p.shape[1])
        p.copy_(((torch.rand(p.shape, generator=g) * 2 - 1) * bound * math.sqrt(3.0)).to(p.device))
    elif b_std > 0:
        p.copy_(torch.empty(p.shape).normal_(0, b_std, generator=g).to(p.device))
    else:
        p.zero_()


def merge_lora(model: nn.Module) -> int:
    n = 0
    for m in model.modules():
        if isinstance(m, LoraLinear):
            m.merge()
            n += 1
        elif isinstance(getattr(m, "lora", None), ExpertsLoRA):
            m.lora.merge_into(m)
            n += 1
    return n


def lora_state_dict_peft(named_full_tensors: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """In-memory names (``...qkv_proj.lora_A.q_proj``) -> PEFT names
    (``base_model.model.model...q_proj.lora_A.weight``)."""
    out = {}
    for name, t in named_full_tensors.items():
        if name.endswith("_lora_A") or name.endswith("_lora_B"):
            # stacked expert adapters -> one PEFT pair per expert: A [r, in], B [out, r]; a factor shared by
            # all experts (hybrid-shared adapters) is written under every expert
            mod, leaf = name.rsplit(".", 1)                      # ...mlp.experts.lora , gate_proj_lora_A
            proj, kind = leaf.rsplit("_lora_", 1)
            experts = mod.rsplit(".", 1)[0]
            partner = named_full_tensors.get(f"{mod}.{proj}_lora_{'B' if kind == 'A' else 'A'}")
            E = max(t.shape[0], partner.shape[0] if partner is not None else 1)
            for e in range(E):
                out[f"base_model.model.model.{experts}.{e}.{proj}.lora_{kind}.weight"] = t[e if t.shape[0] > 1 else 0].t().contiguous()
            continue
        if ".lora_A." not in name and ".lora_B." not in name:
            continue
        mod, kind, part = name.rsplit(".", 2)
        parent = mod.rsplit(".", 1)[0]
        prefix = "base_model.model." + ("" if parent.startswith("lm_head") else "model.")
        out[f"{prefix}{parent}.{part}.{kind}.weight"] = t
    return out


def slice_to_rank(name: str, t: torch.Tensor, rank: int) -> torch.Tensor:
    """The first ``rank`` rank components of an adapter matrix in its in-memory layout (dense A [R, in],
    B [out, R]; stacked experts A [E, in, R], B [E, R, out])."""
    if name.endswith("_lora_A"):
        return t[..., :rank]
    if name.endswith("_lora_B"):
        return t[:, :rank]
    if ".lora_A." in name:
        return t[:rank]
    if ".lora_B." in name:
        return t[:, :rank]
    return t


def save_lora_checkpoint(engine, out_dir: str, base_model_name: str = "", rank: Optional[int] = None,
                         alpha: Optional[float] = None) -> None:
    """PEFT directory: ``adapter_model.safetensors`` + ``adapter_config.json``.  ``rank`` / ``alpha``: the
    active session's own (an adapter of lower rank than the storage is written at its rank: its remaining
    components are zero)."""
    from safetensors.torch import save_file
    tensors = {n: t.detach().to(torch.bfloat16).cpu().contiguous()
               for n, t in engine.iter_full_tensors("master") if ".lora_" in n or "_lora_" in n}
    if engine.ps.rank != 0:
        return
    cfg = dict(getattr(engine.model, "_xb_lora_config", {}))
    if rank is not None and rank < cfg.get("r", rank):
        tensors = {n: slice_to_rank(n, t, rank).contiguous() for n, t in tensors.items()}
        cfg["r"] = int(rank)
    if alpha is not None:
        cfg["lora_alpha"] = alpha
    os.makedirs(out_dir, exist_ok=True)
    save_file(lora_state_dict_peft(tensors), os.path.join(out_dir, "adapter_model.safetensors"),
              metadata={"format": "pt"})
    cfg.update({"peft_type": "LORA", "task_type": "CAUSAL_LM", "base_model_name_or_path": base_model_name,
                "bias": "none", "lora_dropout": 0.0, "inference_mode": True, "fan_in_fan_out": False})
    with open(os.path.join(out_dir, "adapter_config.json"), "w") as f:
        json.dump(cfg, f, indent=2)


def merged_weight_view(engine):
    """``fn(name, full_weight) -> full_weight`` with the active adapter folded in
    (``W + scaling * B A``, per output slice for fused projections, per expert for stacked experts), or
    None for a model without adapters.  Building it gathers the adapter matrices (a collective: every
    rank calls it); the frozen base weights in the engine are not touched, so training goes on with the
    adapter separate.  This is what an inference engine is sent for a LoRA policy
    (src/xorl/trainers/training_utils.py:346-372 merges in place and unmerges afterwards)."""
    mods = {n: m for n, m in engine.model.named_modules()
            if isinstance(m, LoraLinear) or isinstance(getattr(m, "lora", None), ExpertsLoRA)}
    if not mods:
        return None
    factors = {n: t.float() for n, t in engine.iter_full_tensors("master") if ".lora_" in n or "_lora_" in n}

    def fold(name: str, w: torch.Tensor) -> torch.Tensor:
        mod, _, leaf = name.rpartition(".")
        m = mods.get(mod)
        if isinstance(m, LoraLinear) and leaf == "weight":
            out = w.float().clone()
            for part, s, e in m.slices:
                out[s:e] += (factors[f"{mod}.lora_B.{part}"] @ factors[f"{mod}.lora_A.{part}"]).to(out.device) * m.scaling
            return out.to(w.dtype)
        lora = getattr(m, "lora", None) if m is not None else None
        if isinstance(lora, ExpertsLoRA) and leaf in ("gate_up_proj", "down_proj"):
            out = w.float().clone()
            I = out.shape[1] if leaf == "down_proj" else out.shape[2] // 2
            for p in lora.targets:
                if (p == "down_proj") != (leaf == "down_proj"):
                    continue
                fa, fb = factors[f"{mod}.lora.{p}_lora_A"], factors[f"{mod}.lora.{p}_lora_B"]
                delta = torch.bmm(fa.expand(out.shape[0], -1, -1), fb.expand(out.shape[0], -1, -1)).to(out.device)
                delta = delta * lora.scaling
                if p == "gate_proj":
                    out[:, :, :I] += delta
                elif p == "up_proj":
                    out[:, :, I:] += delta
                else:
                    out += delta
            return out.to(w.dtype)
        return w
    return fold


@contextmanager
def adapters_disabled(model: nn.Module):
    """Inside the block every LoRA module computes its frozen base projection only: the forward pass
    of the reference policy that the adapters started from (reference log-probabilities for KL
    penalties, src/xorl/server/runner/model_runner.py ``forward`` with the adapter detached)."""
    mods = [m for m in model.modules() if isinstance(m, (LoraLinear, ExpertsLoRA))]
    prev = [getattr(m, "enabled", True) for m in mods]
    for m in mods:
        m.enabled = False
    try:
        yield len(mods)
    finally:
        for m, e in zip(mods, prev):
            m.enabled = e
