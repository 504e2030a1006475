"""Model zoo: configuration loading, family registry, model construction."""
from __future__ import annotations

import os
from typing import Any

from .config import PRESETS, ModelConfig, preset  # noqa: F401
from .registry import MODEL_REGISTRY, get_model_class  # noqa: F401


def build_model_config(model_args) -> ModelConfig:
    """From ``model.config_path`` / ``model.model_path`` (a directory with config.json, a json
    file, or the name of a built-in preset) plus ``model.foundation`` overrides."""
    src = model_args.config_path or model_args.model_path
    if src is None:
        raise ValueError("model.config_path or model.model_path is required")
    key = str(src).lower().split("/")[-1]
    if os.path.exists(src):
        cfg = ModelConfig.from_pretrained(src)
    elif key in PRESETS:
        cfg = preset(key)
    else:
        raise FileNotFoundError(f"no config.json at {src!r} and no preset named {key!r} "
                                f"(presets: {sorted(PRESETS)})")
    for k, v in (model_args.foundation or {}).items():
        if hasattr(cfg, k):
            setattr(cfg, k, v)
        else:
            cfg.extra[k] = v
    return cfg


def build_model(cfg: ModelConfig, args: Any = None, device="meta", dtype=None, **stage_kw):
    """Instantiates the family's model class (parameters on ``device``; ``meta`` by default, the
    ZeRO engine materialises them shard by shard)."""
    cls = get_model_class(cfg)
    model = cls(cfg, dtype=dtype, device=device, **stage_kw)
    if args is not None:
        from ..adapters import apply_adapters
        apply_adapters(model, cfg, args)
    return model
