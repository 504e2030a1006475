"""What a training session asked for: the adapter shape and the optimizer, normalised once when the
session is created, stored next to its checkpoints, and read back when the session is restored
(src/xorl/server/session_spec.py).

A spec is a plain JSON-able dict
``{"version": 1, "base_model": ..., "lora": {"rank", "alpha", "target_modules", "dropout"},
"optimizer": {"type", "learning_rate", "weight_decay", "betas", "eps", "dtype", "kwargs"}}``.
Requests may spell keys the PEFT way (``r``, ``lora_alpha``); unknown optimizer types, ranks above
the server's limit and non-finite numbers are refused here, before any GPU work.
"""
from __future__ import annotations

import copy
import json
import math
import os
from typing import Any, Dict, Optional, Sequence

SPEC_FILE = "session_spec.json"
SPEC_VERSION = 1
OPTIMIZER_TYPES = ("adamw", "anyprecision_adamw", "sgd", "signsgd", "distsignsgd", "muon")
_LORA_ALIASES = {"r": "rank", "lora_rank": "rank", "lora_alpha": "alpha", "lora_dropout": "dropout",
                 "lora_target_modules": "target_modules"}


def _finite(x, name: str, lo: float = 0.0) -> float:
    v = float(x)
    if not math.isfinite(v) or v < lo:
        raise ValueError(f"{name} must be a finite number >= {lo}, got {x!r}")
    return v


def normalize_lora(raw: Optional[Dict[str, Any]], *, default_rank: int, default_alpha: float, max_rank: int,
                   server_targets: Optional[Sequence[str]] = None) -> Dict[str, Any]:
    cfg = {_LORA_ALIASES.get(k, k): v for k, v in (raw or {}).items()}
    unknown = set(cfg) - {"rank", "alpha", "target_modules", "dropout"}
    if unknown:
        raise ValueError(f"unknown LoRA settings: {sorted(unknown)}")
    rank = int(cfg.get("rank", default_rank))
    if not 1 <= rank <= max_rank:
        raise ValueError(f"LoRA rank {rank} outside [1, {max_rank}]")
    targets = list(cfg.get("target_modules") or server_targets or [])
    if server_targets is not None and not set(targets) <= set(server_targets):
        raise ValueError(f"target modules {sorted(set(targets) - set(server_targets))} are not adapted by this server")
    return {"rank": rank, "alpha": _finite(cfg.get("alpha", default_alpha), "alpha"),
            "target_modules": sorted(targets), "dropout": _finite(cfg.get("dropout", 0.0), "dropout")}


def normalize_optimizer(raw: Optional[Dict[str, Any]], *, default_type: str = "adamw", default_lr: float = 1e-4,
                        default_weight_decay: float = 0.0, default_dtype: str = "bf16",
                        default_betas=(0.9, 0.95), default_eps: float = 1e-12,
                        default_kwargs: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    cfg = dict(raw or {})
    kind = str(cfg.pop("type", cfg.pop("optimizer", default_type))).lower()
    if kind not in OPTIMIZER_TYPES:
        raise ValueError(f"unknown optimizer type {kind!r}; one of {OPTIMIZER_TYPES}")
    betas = tuple(float(b) for b in cfg.pop("betas", default_betas))
    if len(betas) != 2 or not all(0.0 <= b < 1.0 for b in betas):
        raise ValueError(f"betas must be two numbers in [0, 1), got {betas}")
    out = {"type": kind,
           "learning_rate": _finite(cfg.pop("learning_rate", cfg.pop("lr", default_lr)), "learning_rate"),
           "weight_decay": _finite(cfg.pop("weight_decay", default_weight_decay), "weight_decay"),
           "betas": list(betas), "eps": _finite(cfg.pop("eps", default_eps), "eps"),
           "dtype": str(cfg.pop("dtype", cfg.pop("optimizer_dtype", default_dtype))),
           "kwargs": {**(default_kwargs or {}), **cfg.pop("kwargs", {})}}
    if out["dtype"] not in ("bf16", "fp32"):
        raise ValueError(f"optimizer dtype must be bf16 or fp32, got {out['dtype']!r}")
    if cfg:
        raise ValueError(f"unknown optimizer settings: {sorted(cfg)}")
    return out


def normalize_session_spec(*, base_model: str, lora: Optional[Dict[str, Any]], optimizer: Optional[Dict[str, Any]],
                           lora_defaults: Dict[str, Any], optimizer_defaults: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    return {"version": SPEC_VERSION, "base_model": str(base_model),
            "lora": normalize_lora(lora, **lora_defaults),
            "optimizer": normalize_optimizer(optimizer, **(optimizer_defaults or {}))}


def optimizer_build_kwargs(opt: Dict[str, Any]) -> Dict[str, Any]:
    """Keyword arguments of ``xorl_b200.optim.build_optimizer`` for a normalised optimizer spec."""
    return dict(lr=opt["learning_rate"], betas=tuple(opt["betas"]), eps=opt["eps"], weight_decay=opt["weight_decay"],
                optimizer_type=opt["type"], optimizer_dtype=opt["dtype"], optimizer_kwargs=copy.deepcopy(opt["kwargs"]))


def write_session_spec(directory: str, spec: Dict[str, Any]) -> str:
    os.makedirs(directory, exist_ok=True)
    path = os.path.join(directory, SPEC_FILE)
    tmp = path + ".tmp"
    with open(tmp, "w") as f:
        json.dump(spec, f, indent=2, sort_keys=True)
    os.replace(tmp, path)
    return path


def read_session_spec(directory: str, fallback: Optional[Dict[str, Any]] = None) -> Dict[str, Any]:
    """The spec stored with a checkpoint; a PEFT ``adapter_config.json`` is enough to rebuild the
    adapter part when an older checkpoint has no spec file."""
    path = os.path.join(directory, SPEC_FILE)
    if os.path.exists(path):
        with open(path) as f:
            spec = json.load(f)
        if spec.get("version") != SPEC_VERSION:
            raise ValueError(f"session spec version {spec.get('version')} is not supported")
        return spec
    peft = os.path.join(directory, "adapter_config.json")
    if os.path.exists(peft) and fallback is not None:
        with open(peft) as f:
            a = json.load(f)
        spec = copy.deepcopy(fallback)
        spec["lora"].update(rank=int(a.get("r", spec["lora"]["rank"])), alpha=float(a.get("lora_alpha", spec["lora"]["alpha"])),
                            target_modules=sorted(a.get("target_modules") or spec["lora"]["target_modules"]))
        return spec
    if fallback is not None:
        return copy.deepcopy(fallback)
    raise FileNotFoundError(path)
