"""Quantisation-aware RL: the policy trains on the numerics of the quantised weights (and, optionally,
activations) that the inference engine will run, while the master weights stay in full precision.

Every selected linear (and, for nvfp4, every stacked-experts module) computes with
``x + (dequantise(quantise(x)) - x).detach()``: the forward sees the quantisation grid, the backward is
the identity (straight-through), so the optimizer keeps moving the full-precision masters.  Two grids
(src/xorl/qarl/fake_quant.py, moe_experts.py; src/xorl/ops/quantize/nvfp4_fake_quant.py):

* ``fp8_e4m3`` -- weights in 2-D blocks (default 128 x 128) with one scale per block, activations with
  one dynamic scale per tensor; dense models only;
* ``nvfp4`` -- e2m1 values in groups of 16 along the contraction dimension with an e4m3 scale per group
  and one fp32 scale per tensor; weight-only unless ``activation: true``; also covers MoE experts.

Each wrapped module records the last absolute maxima it saw and how often it ran; a calibration pass
(``train.qarl_calib_data``) warms these numbers up before training and writes them out, and the weight
sync to the inference engine exports exactly the wrapped weights in the matching format
(``sync_quantization_config``)."""
from __future__ import annotations

import fnmatch
import json
import os
from typing import Any, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple

import torch
from torch import nn

from ..models.layers import Linear
from ..ops import gemm as gemm_ops
from ..ops import quantize as Q

FP8_NAMES = ("fp8", "fp8_e4m3", "e4m3", "fp8_default_cfg")
NVFP4_NAMES = ("nvfp4",)
NVFP4_GROUP = 16                      # the block size every nvfp4 consumer (export, serving kernels) assumes
_CFG_KEYS = {"format", "quant_method", "weight", "activation", "dynamic", "weight_block_size", "group_size"}


def _format_of(name: str) -> str:
    n = str(name).strip().lower()
    if n in NVFP4_NAMES:
        return "nvfp4"
    if n in FP8_NAMES:
        return "fp8_e4m3"
    raise ValueError(f"qarl_quant_cfg format {name!r} is not one of {FP8_NAMES + NVFP4_NAMES}")


def normalize_quant_cfg(cfg: Optional[Any], default_format: str = "fp8") -> Dict[str, Any]:
    """``None`` / an alias string / a mapping -> the full configuration.  fp8 quantises weights and
    activations by default, nvfp4 weights only.  Static (calibrated, frozen) scales do not exist: the
    scales are recomputed from the live tensors every forward."""
    if cfg is None:
        cfg = default_format
    if isinstance(cfg, str):
        cfg = {"format": cfg}
    if not isinstance(cfg, Mapping):
        raise ValueError(f"qarl_quant_cfg must be a mapping, a format name or null, got {type(cfg).__name__}")
    unknown = set(cfg) - _CFG_KEYS
    if unknown:
        raise ValueError(f"unknown qarl_quant_cfg keys {sorted(unknown)}")
    fmt = _format_of(cfg.get("format", cfg.get("quant_method", default_format)))
    if not bool(cfg.get("dynamic", True)):
        raise ValueError("qarl_quant_cfg.dynamic=false (static scales) is not available; scales are dynamic")
    if fmt == "nvfp4":
        group = cfg.get("group_size", NVFP4_GROUP)
        if group != NVFP4_GROUP:
            raise ValueError(f"qarl_quant_cfg.group_size must be {NVFP4_GROUP} for nvfp4, got {group!r}")
        return {"format": fmt, "weight": bool(cfg.get("weight", True)), "activation": bool(cfg.get("activation", False)),
                "dynamic": True, "group_size": NVFP4_GROUP}
    block = cfg.get("weight_block_size", (128, 128))
    if not (isinstance(block, (list, tuple)) and len(block) == 2
            and all(isinstance(b, int) and not isinstance(b, bool) and b > 0 for b in block)):
        raise ValueError("qarl_quant_cfg.weight_block_size must be two positive integers")
    return {"format": fmt, "weight": bool(cfg.get("weight", True)), "activation": bool(cfg.get("activation", True)),
            "dynamic": True, "weight_block_size": [int(block[0]), int(block[1])]}


def unsupported_scope(model_config: Any = None, selectors: Iterable[str] = ()) -> Optional[str]:
    """Why fake quantisation cannot cover this model (None when it can): multi-token-prediction heads and
    state-space (Mamba) mixers are outside its scope."""
    def get(c, k):
        return c.get(k) if isinstance(c, Mapping) else getattr(c, k, None)

    for c in (model_config, get(model_config, "text_config") if model_config is not None else None):
        if c is None:
            continue
        for k in ("mtp_num_hidden_layers", "mtp_num_layers", "num_nextn_predict_layers"):
            v = get(c, k)
            if isinstance(v, int) and not isinstance(v, bool) and v > 0:
                return f"QARL does not cover multi-token-prediction layers ({k}={v})"
        for k in ("model_type", "family"):
            v = get(c, k)
            if isinstance(v, str) and ("mamba" in v.lower() or "nemotron_h" in v.lower()):
                return f"QARL does not cover state-space mixers ({k}={v})"
    for s in selectors:
        parts = [p.lower() for p in str(s).replace("/", ".").split(".") if p]
        if any(p == "mtp" or p.startswith("mtp_") or p == "nextn" or p.startswith("nextn_") for p in parts):
            return f"QARL does not cover multi-token-prediction layers (module selector {s!r})"
    return None


# ---------------------------------------------------------------------------------------------
# grids
# ---------------------------------------------------------------------------------------------
def _ste(x: torch.Tensor, dq: torch.Tensor) -> torch.Tensor:
    return x + (dq.to(x.dtype) - x).detach()


def fake_quant_fp8_blocks(w: torch.Tensor, block: Sequence[int] = (128, 128)) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 with one scale per ``block`` of a 2-D weight.  Returns (straight-through tensor, scales)."""
    with torch.no_grad():
        br, bc = int(block[0]), int(block[1])
        if br == bc:
            q, s = Q.block_fp8_quantize_128x128(w, br)
            dq = Q.block_fp8_dequantize_128x128(q, s, br, w.dtype)
        else:
            N, K = w.shape
            nb, kb = -(-N // br), -(-K // bc)
            wp = torch.zeros(nb * br, kb * bc, dtype=torch.float32, device=w.device)
            wp[:N, :K] = w.float()
            blk = wp.reshape(nb, br, kb, bc)
            s = (blk.abs().amax((1, 3)) / Q.FP8_MAX).clamp_min(1e-12)
            qv = (blk / s[:, None, :, None]).clamp(-Q.FP8_MAX, Q.FP8_MAX).to(torch.float8_e4m3fn).float()
            dq = (qv * s[:, None, :, None]).reshape(nb * br, kb * bc)[:N, :K]
    return _ste(w, dq), s


def fake_quant_fp8_tensor(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """e4m3 with one dynamic scale for the whole tensor (activations)."""
    with torch.no_grad():
        s = (x.float().abs().amax() / Q.FP8_MAX).clamp_min(1e-12)
        dq = (x.float() / s).clamp(-Q.FP8_MAX, Q.FP8_MAX).to(torch.float8_e4m3fn).float() * s
    return _ste(x, dq), s


def fake_quant_nvfp4(w: torch.Tensor, group: int = NVFP4_GROUP, dim: int = -1) -> torch.Tensor:
    """nvfp4 with the groups of ``group`` elements laid along ``dim`` (the contraction dimension)."""
    with torch.no_grad():
        wt = w.transpose(dim, -1) if dim not in (-1, w.dim() - 1) else w
        K = wt.shape[-1]
        pad = (-K) % group
        wp = torch.nn.functional.pad(wt, (0, pad)) if pad else wt
        wp = wp.contiguous()
        p, s, g = Q.nvfp4_quantize(wp, group)
        dq = Q.nvfp4_dequantize(p, s, g, wp.shape, group, w.dtype)[..., :K]
        if wt is not w:
            dq = dq.transpose(dim, -1)
    return _ste(w, dq)


def fake_quant(w: torch.Tensor, fmt: str) -> torch.Tensor:
    """Weight fake quantisation by format name (``fp8`` / ``nvfp4`` / ``bf16`` = none)."""
    if fmt in ("bf16", None):
        return w
    return fake_quant_nvfp4(w) if _format_of(fmt) == "nvfp4" else fake_quant_fp8_blocks(w)[0]


# ---------------------------------------------------------------------------------------------
# modules
# ---------------------------------------------------------------------------------------------
class FakeQuantLinear(nn.Module):
    """A ``Linear`` whose forward runs on the fake-quantised weight (and input).  The parameter objects
    are the base layer's own, so names, ZeRO shards, optimizer state and checkpoints do not change."""

    def __init__(self, base: Linear, cfg: Mapping[str, Any]):
        super().__init__()
        self.in_features, self.out_features = base.in_features, base.out_features
        self.weight, self.bias = base.weight, base.bias
        self.cfg = dict(cfg)
        self.fmt = cfg["format"]
        self.stats: Dict[str, Any] = {"forward_count": 0, "input_amax": None, "weight_amax": None,
                                      "input_scale": None, "weight_scale_shape": None}

    def forward(self, x):
        st = self.stats
        st["forward_count"] += 1
        with torch.no_grad():                               # device scalars, no host sync on the step path
            st["input_amax"] = x.detach().abs().amax() if x.numel() else None
            st["weight_amax"] = self.weight.detach().abs().amax()
        w, xin = self.weight, x
        if self.fmt == "nvfp4":
            if self.cfg["weight"]:
                w = fake_quant_nvfp4(w, self.cfg["group_size"])
            if self.cfg["activation"]:
                xin = fake_quant_nvfp4(x, self.cfg["group_size"])
        else:
            if self.cfg["weight"]:
                w, ws = fake_quant_fp8_blocks(w, self.cfg["weight_block_size"])
                st["weight_scale_shape"] = tuple(ws.shape)
            if self.cfg["activation"] and x.numel():
                xin, st["input_scale"] = fake_quant_fp8_tensor(x)
        return gemm_ops.linear(xin, w, self.bias)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}, {self.cfg}"


_FAKE_QUANT_EXPERT_CLASSES: Dict[type, type] = {}


def fake_quantize_experts_(experts: nn.Module, cfg: Mapping[str, Any]) -> None:
    """Stacked experts (``gate_up_proj [E, H, 2I]``, ``down_proj [E, I, H]``; contraction along dim 1):
    the attributes return the nvfp4 fake-quantised tensors, so the local, all-to-all and fused-dispatch
    paths all compute on them; the parameters themselves (and so shards, expert-parallel slices and
    checkpoints) stay as they are.  The per-expert scales need no communication: each rank quantises the
    experts it holds.  With ``activation`` the tokens entering the experts are fake-quantised too."""
    cls = type(experts)
    if cls not in _FAKE_QUANT_EXPERT_CLASSES:
        def prop(name):
            def get(self):
                p = self._parameters[name]
                c = self._qarl_cfg
                return fake_quant_nvfp4(p, c["group_size"], dim=1) if c["weight"] else p
            return property(get)
        _FAKE_QUANT_EXPERT_CLASSES[cls] = type("FakeQuant" + cls.__name__, (cls,),
                                               {"gate_up_proj": prop("gate_up_proj"), "down_proj": prop("down_proj")})
    experts._qarl_cfg = dict(cfg)
    experts.__class__ = _FAKE_QUANT_EXPERT_CLASSES[cls]


def _selected(name: str, patterns: Sequence[str]) -> bool:
    short = name.rsplit(".", 1)[-1]
    return any(fnmatch.fnmatch(name, p) or fnmatch.fnmatch(short, p) or p in name.split(".") for p in patterns)


def inject_fake_quant(model: nn.Module, train_args) -> List[str]:
    """Wraps the selected linears (``qarl_target_modules`` / ``qarl_exclude_modules``: names or glob
    patterns on the full or the last name; the lm-head is never wrapped) and, for nvfp4, the stacked
    experts.  ``qarl_quant_cfg`` picks the grid; without it the grid follows ``qarl_sync_format``."""
    cfg = normalize_quant_cfg(getattr(train_args, "qarl_quant_cfg", None),
                              default_format=getattr(train_args, "qarl_sync_format", "fp8"))
    targets = list(getattr(train_args, "qarl_target_modules", None) or [])
    exclude = list(getattr(train_args, "qarl_exclude_modules", None) or []) + ["lm_head"]
    why = unsupported_scope(getattr(model, "config", None), targets + exclude)
    if why:
        raise ValueError(why)
    from ..models.moe import Experts
    experts = [(n, m) for n, m in model.named_modules() if isinstance(m, Experts)]
    if experts and cfg["format"] != "nvfp4":
        raise ValueError("QARL on a MoE model needs the nvfp4 format: fp8 fake quantisation covers dense models only")
    wrapped: List[str] = []
    for pname, parent in list(model.named_modules()):
        for cname, child in list(parent.named_children()):
            full = f"{pname}.{cname}" if pname else cname
            if type(child) is not Linear or _selected(full, exclude) or (targets and not _selected(full, targets)):
                continue
            if cname == "gate" and any(pname == n.rsplit(".", 1)[0] for n, _ in experts):
                continue                                                  # MoE routers stay exact
            setattr(parent, cname, FakeQuantLinear(child, cfg))
            wrapped.append(full)
    expert_names = []
    for name, m in experts:
        if _selected(name, exclude) or (targets and not _selected(name, targets)):
            continue
        fake_quantize_experts_(m, cfg)
        expert_names.append(name)
    model._xb_qarl_config = {"quant_cfg": cfg, "linears": wrapped, "experts": expert_names,
                             "target_modules": targets, "exclude_modules": exclude}
    return wrapped + expert_names


def summarize(model: nn.Module) -> Dict[str, Any]:
    """What the wrapped modules have seen (reads device scalars: call it off the step path)."""
    out: Dict[str, Any] = {"enabled": False, "linear_count": 0, "modules": {}}
    for name, m in model.named_modules():
        if isinstance(m, FakeQuantLinear):
            st = m.stats
            f = lambda v: None if v is None else float(v)
            out["modules"][name] = {"forward_count": int(st["forward_count"]), "input_amax": f(st["input_amax"]),
                                    "weight_amax": f(st["weight_amax"]), "input_scale": f(st["input_scale"]),
                                    "weight_scale_shape": st["weight_scale_shape"]}
    out["linear_count"] = len(out["modules"])
    out["experts"] = list(getattr(model, "_xb_qarl_config", {}).get("experts", []))
    out["enabled"] = bool(out["modules"] or out["experts"])
    return out


# ---------------------------------------------------------------------------------------------
# calibration (train.qarl_calib_data / qarl_calib_size / qarl_quant_sequence_length)
# ---------------------------------------------------------------------------------------------
def load_calibration_batches(path: str, size: int = 0, sequence_length: Optional[int] = None) -> List[torch.Tensor]:
    """Token-id batches ``[rows, tokens]`` from a ``.json`` (a list, or a mapping with ``input_ids`` /
    ``samples`` / ``batches``), ``.jsonl`` (one batch or ``{"input_ids": ...}`` per line) or ``.pt`` file;
    at most ``size`` batches (0 = all), each cut to ``sequence_length`` tokens."""
    if size < 0:
        raise ValueError("qarl_calib_size must be non-negative")
    if sequence_length is not None and sequence_length <= 0:
        raise ValueError("qarl_quant_sequence_length must be positive when set")
    ext = os.path.splitext(path)[1].lower()
    if ext in (".pt", ".pth"):
        payload = torch.load(path, map_location="cpu", weights_only=True)
    elif ext == ".jsonl":
        with open(path, encoding="utf-8") as f:
            payload = [json.loads(line) for line in f if line.strip()]
    elif ext == ".json":
        with open(path, encoding="utf-8") as f:
            payload = json.load(f)
    else:
        raise ValueError("qarl_calib_data must be a .json, .jsonl, .pt or .pth file")
    if isinstance(payload, Mapping):
        for k in ("batches", "samples", "input_ids"):
            if k in payload:
                payload = payload[k]
                break
        else:
            raise ValueError("calibration mapping needs one of: batches, samples, input_ids")
    if isinstance(payload, torch.Tensor):
        payload = [payload]
    batches = []
    for raw in list(payload)[: size or None]:
        ids = raw["input_ids"] if isinstance(raw, Mapping) else raw
        t = (ids.detach().cpu() if isinstance(ids, torch.Tensor) else torch.as_tensor(ids)).long()
        t = t[None] if t.dim() == 1 else t
        if t.dim() != 2:
            raise ValueError(f"calibration token ids must be 1-D or 2-D, got shape {tuple(t.shape)}")
        batches.append(t[:, :sequence_length] if sequence_length else t)
    if not batches:
        raise ValueError("calibration data holds no batches")
    return batches


def calibrate(forward, model: nn.Module, path: str, size: int = 0, sequence_length: Optional[int] = None,
              device=None) -> Dict[str, Any]:
    """Runs the calibration batches through ``forward(input_ids)`` without gradients (this fills the
    wrapped modules' statistics and is a pre-flight of every fake-quant path) and returns the summary."""
    batches = load_calibration_batches(path, size, sequence_length)
    with torch.no_grad():
        for b in batches:
            forward(b.to(device) if device is not None else b)
    out = summarize(model)
    out["calibration_batches"] = len(batches)
    out["calibration_samples"] = int(sum(b.shape[0] for b in batches))
    return out


# ---------------------------------------------------------------------------------------------
# weight sync
# ---------------------------------------------------------------------------------------------
def sync_quantization_config(model: nn.Module, base: Optional[Mapping[str, Any]] = None) -> Optional[Dict[str, Any]]:
    """Quantisation block of the weight sync for a fake-quantised model: the receiver gets exactly the
    wrapped weights in the trained grid, every other 2-D weight in the source precision
    (``modules_to_not_convert``) (src/xorl/qarl/sync.py:53-101).  None when the model is not wrapped and
    no base configuration is given."""
    info = getattr(model, "_xb_qarl_config", None)
    if not info or not (info["linears"] or info["experts"]):
        return dict(base) if base is not None else None
    cfg = info["quant_cfg"]
    out = dict(base or {})
    if cfg["format"] == "nvfp4":
        out.setdefault("quant_method", "nvfp4")
        out.setdefault("group_size", cfg["group_size"])
        if out["group_size"] != cfg["group_size"]:
            raise ValueError(f"sync group_size {out['group_size']} differs from the trained {cfg['group_size']}")
    else:
        out.setdefault("quant_method", "fp8")
        out.setdefault("fmt", "e4m3")
        out.setdefault("activation_scheme", "dynamic")
        block = list(cfg["weight_block_size"])
        if "weight_block_size" in out and list(out["weight_block_size"]) != block:
            raise ValueError(f"sync weight_block_size {list(out['weight_block_size'])} differs from the trained {block}")
        out["weight_block_size"] = block
    wrapped = set(info["linears"]) | set(info["experts"])
    skipped, seen = [], set()
    for n, p in model.named_parameters():
        mod = n.rsplit(".", 1)[0]
        if p.dim() >= 2 and mod not in wrapped and mod not in seen:
            seen.add(mod)
            skipped.append(mod)
    out["modules_to_not_convert"] = list(out.get("modules_to_not_convert") or []) + skipped
    out["qarl"] = {"enabled": True, "folded_modules": sorted(wrapped), "source": "fake_quant"}
    return out
