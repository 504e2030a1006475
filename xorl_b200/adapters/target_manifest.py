"""Strict coverage manifests for LoRA targets.

``lora_target_modules`` names leaves (``q_proj``, ``down_proj``); which and how many adapters that gives
depends on the model.  A manifest pins the result down: the leaf list plus, per name pattern, how many
adapter units the injected model must have and at which rank.  It is checked on the model instance right
after injection, before any sharding or training step (src/xorl/lora/target_manifest.py).

    {"schema_version": 1,
     "target_modules": ["q_proj", "v_proj"],
     "expected_modules": [{"pattern": "model.layers.*.self_attn.q_proj", "count": 36, "rank": 16},
                          {"pattern": "model.layers.*.self_attn.v_proj", "count": 36}],
     "allow_unlisted": false}

Adapter units are named as the Hugging Face module they adapt: a fused projection that carries one
adapter per output slice counts once per slice (``model.layers.3.self_attn.q_proj``), a stacked-experts
module once (``model.layers.3.mlp.experts``)."""
from __future__ import annotations

import fnmatch
import json
from typing import Any, Dict, Iterable, List, Mapping, Optional, Tuple, Union

from torch import nn

SCHEMA_VERSION = 1
Manifest = Union[Mapping[str, Any], str, None]


def load_manifest(value: Manifest) -> Optional[Dict[str, Any]]:
    """A mapping, a path to a JSON file, or None.  Raises on anything that is not a version-1 manifest."""
    if value is None or value == "":
        return None
    if isinstance(value, str):
        with open(value) as f:
            m = json.load(f)
    elif isinstance(value, Mapping):
        m = dict(value)
    else:
        raise TypeError(f"lora_target_manifest must be a mapping, a path or null, got {type(value).__name__}")
    if type(m.get("schema_version")) is not int or m["schema_version"] != SCHEMA_VERSION:
        raise ValueError(f"lora target manifest schema_version {m.get('schema_version')!r} is not {SCHEMA_VERSION}")
    if "allow_unlisted" in m and type(m["allow_unlisted"]) is not bool:
        raise ValueError("lora target manifest: allow_unlisted must be true or false")
    targets = m.get("target_modules")
    if not (isinstance(targets, list) and targets and all(isinstance(t, str) for t in targets)):
        raise ValueError("lora target manifest: target_modules must be a non-empty list of names")
    entries = m.get("expected_modules")
    if not (isinstance(entries, list) and entries):
        raise ValueError("lora target manifest: expected_modules must be a non-empty list")
    for e in entries:
        if not (isinstance(e, dict) and isinstance(e.get("pattern"), str)):
            raise ValueError(f"lora target manifest: bad expected_modules entry {e!r}")
        if type(e.get("count")) is not int or e["count"] < 0:
            raise ValueError(f"lora target manifest: count must be a non-negative integer in {e!r}")
        if e.get("rank") is not None and (type(e["rank"]) is not int or e["rank"] <= 0):
            raise ValueError(f"lora target manifest: rank must be a positive integer or null in {e!r}")
    return m


def resolve_targets(target_modules: Optional[Iterable[str]], manifest: Manifest
                    ) -> Tuple[Optional[List[str]], Optional[Dict[str, Any]]]:
    """The leaf list to inject with.  A manifest's list wins; a configured list that differs from it is an error."""
    m = load_manifest(manifest)
    if m is None:
        return (None if target_modules is None else list(target_modules)), None
    if target_modules is not None and set(target_modules) != set(m["target_modules"]):
        raise ValueError(f"lora_target_modules {sorted(target_modules)} differ from the manifest's "
                         f"{sorted(m['target_modules'])}")
    return list(m["target_modules"]), m


def adapter_units(model: nn.Module, prefix: str = "model.") -> Dict[str, int]:
    """{Hugging Face module name: rank} of every adapter the model carries."""
    from .lora import ExpertsLoRA, LoraLinear
    out: Dict[str, int] = {}
    for name, m in model.named_modules():
        if isinstance(m, LoraLinear):
            parent = name.rsplit(".", 1)[0] if "." in name else ""
            root = "" if name.startswith("lm_head") else prefix
            for part, _s, _e in m.slices:                     # slice names are the Hugging Face leaf names
                out[f"{root}{parent + '.' if parent else ''}{part}"] = int(m.rank)
        elif isinstance(getattr(m, "lora", None), ExpertsLoRA):
            out[f"{prefix}{name}"] = int(m.lora.rank)
    return out


def validate(model: nn.Module, manifest: Manifest) -> Dict[str, int]:
    """Raises ValueError listing every mismatch: a pattern's count or rank, patterns that overlap, adapter
    units no pattern lists (unless ``allow_unlisted``).  Returns the model's adapter units."""
    m = load_manifest(manifest)
    if m is None:
        raise ValueError("no manifest to validate against")
    actual = adapter_units(model)
    seen: set = set()
    errors: List[str] = []
    for e in m["expected_modules"]:
        names = sorted(n for n in actual if fnmatch.fnmatchcase(n, e["pattern"]))
        if len(names) != e["count"]:
            errors.append(f"{e['pattern']!r}: {len(names)} adapter units, the manifest expects {e['count']}")
        if e.get("rank") is not None:
            wrong = {n: actual[n] for n in names if actual[n] != e["rank"]}
            if wrong:
                errors.append(f"{e['pattern']!r}: rank {e['rank']} expected, found {wrong}")
        twice = seen.intersection(names)
        if twice:
            errors.append(f"{e['pattern']!r}: also matched by an earlier pattern: {sorted(twice)}")
        seen.update(names)
    if not m.get("allow_unlisted", False):
        extra = sorted(set(actual) - seen)
        if extra:
            errors.append(f"adapter units no pattern lists: {extra}")
    if errors:
        raise ValueError("lora target manifest check failed: " + "; ".join(errors))
    return actual
