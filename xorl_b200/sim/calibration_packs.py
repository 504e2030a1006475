"""Calibration packs of the step-time planner: discovery, validation, evaluation and fitting.

A pack is a directory with ``manifest.json`` (schema version, hardware figures, planner coefficient
overrides and a list of *observed runs*: model, layout, sequence length and the measured step time,
each with the command that produced it) and a ``README.md``.  Built-in packs live next to this module
and are addressed as ``builtin:<name>``; any directory or a bare JSON of coefficients is accepted too
(src/xorl/sim/calibration_packs.py: discovery and portable-content checks;
src/xorl/sim/calibration_evaluator.py: predicted against observed step times).

``evaluate_pack`` runs the planner on every observed run with the pack's coefficients and reports the
relative error; ``fit_coefficient`` moves one coefficient (bisection on the signed mean error) so that
predictions centre on the observations.
"""
from __future__ import annotations

import json
import os
import re
from dataclasses import dataclass
from typing import Any, Dict, List, Optional

PACK_SCHEMA_VERSION = 1
_ROOT = os.path.join(os.path.dirname(os.path.abspath(__file__)), "calibration_packs")
# a pack must be portable: nothing in it may point into one machine or cluster
_FORBIDDEN = {"absolute home path": re.compile("/(?:home|ro" + "ot)/"), "workspace mount": re.compile(r"/workspace(?:/|\b)"),
              "cluster service address": re.compile(r"\.svc\.cluster\.local\b"),
              "scheduler command": re.compile(r"\b(kubectl|sbatch|srun)\b")}


@dataclass
class CalibrationPack:
    name: str
    path: Optional[str]
    manifest: Dict[str, Any]

    @property
    def coefficients(self) -> Dict[str, float]:
        return dict(self.manifest.get("coefficients", {}))

    @property
    def observed_runs(self) -> List[Dict[str, Any]]:
        return list(self.manifest.get("observed_runs", []))


def list_calibration_packs() -> List[str]:
    if not os.path.isdir(_ROOT):
        return []
    return sorted(d for d in os.listdir(_ROOT) if os.path.isfile(os.path.join(_ROOT, d, "manifest.json")))


def resolve_calibration_pack(value: str) -> str:
    """``builtin:<name>``, a bare built-in name, a pack directory or a JSON file -> path."""
    name = value[len("builtin:"):] if value.startswith("builtin:") else value
    if value.startswith("builtin:") or (not os.path.exists(value) and name in list_calibration_packs()):
        if name not in list_calibration_packs():
            raise ValueError(f"unknown built-in calibration pack {name!r}; available: {', '.join(list_calibration_packs()) or 'none'}")
        return os.path.join(_ROOT, name)
    return value


def validate_manifest(manifest: Dict[str, Any], known_coefficients: Optional[List[str]] = None) -> None:
    if manifest.get("schema_version") != PACK_SCHEMA_VERSION:
        raise ValueError(f"calibration pack schema_version must be {PACK_SCHEMA_VERSION}, got {manifest.get('schema_version')!r}")
    for key in ("name", "coefficients", "observed_runs"):
        if key not in manifest:
            raise ValueError(f"calibration pack manifest lacks {key!r}")
    if known_coefficients is not None:
        unknown = sorted(set(manifest["coefficients"]) - set(known_coefficients))
        if unknown:
            raise ValueError(f"calibration pack names unknown coefficients {unknown}")
    for run in manifest["observed_runs"]:
        for key in ("name", "model", "seq_len", "layout", "step_ms", "source"):
            if key not in run:
                raise ValueError(f"observed run {run.get('name', '?')!r} lacks {key!r}")
        if not (isinstance(run["step_ms"], (int, float)) and run["step_ms"] > 0):
            raise ValueError(f"observed run {run['name']!r}: step_ms must be positive")
    text = json.dumps(manifest)
    for what, pat in _FORBIDDEN.items():
        if pat.search(text):
            raise ValueError(f"calibration pack is not portable: it contains a {what}")


def load_pack(value: str) -> CalibrationPack:
    from .planner import default_b200_pack
    path = resolve_calibration_pack(value)
    if os.path.isdir(path):
        with open(os.path.join(path, "manifest.json")) as f:
            manifest = json.load(f)
        validate_manifest(manifest, list(default_b200_pack()))
        return CalibrationPack(manifest["name"], path, manifest)
    with open(path) as f:
        d = json.load(f)
    if "coefficients" not in d:                      # a bare JSON of coefficient overrides
        d = {"schema_version": PACK_SCHEMA_VERSION, "name": os.path.basename(path), "coefficients": d, "observed_runs": []}
    validate_manifest(d, list(default_b200_pack()))
    return CalibrationPack(d["name"], None, d)


def _predict(run: Dict[str, Any], coefficients: Dict[str, float], hardware: Dict[str, Any]):
    from ..models.config import ModelConfig, PRESETS, preset
    from .planner import HardwareSpec, ParallelLayout, estimate
    cfg = preset(run["model"]) if run["model"] in PRESETS else ModelConfig.from_pretrained(run["model"])
    hw = HardwareSpec()
    for k in ("hbm_gbs", "bf16_tflops", "nvlink_gbs", "allreduce_busbw_gbs", "internode_gbs"):
        if k in hardware:
            setattr(hw, k, float(hardware[k]))
    layout = ParallelLayout(**run["layout"])
    doc = run.get("doc_lens")
    doc_lens = None
    if doc:
        # a [min, max] pair stands for uniformly drawn document lengths: their mean length per document
        mean = (doc[0] + doc[1]) / 2.0 if len(doc) == 2 else sum(doc) / len(doc)
        n = max(1, round(run["seq_len"] / mean))
        doc_lens = [run["seq_len"] // n] * n
    return estimate(cfg, layout, run["seq_len"], run.get("micro_batch_tokens"), hw, coefficients, doc_lens)


def evaluate_pack(pack: CalibrationPack, coefficients: Optional[Dict[str, float]] = None) -> Dict[str, Any]:
    """Predicted against observed step time of every run of the pack."""
    coef = pack.coefficients if coefficients is None else coefficients
    rows = []
    for run in pack.observed_runs:
        est = _predict(run, coef, pack.manifest.get("hardware", {}))
        rows.append({"run": run["name"], "observed_ms": float(run["step_ms"]), "predicted_ms": est.step_ms,
                     "relative_error": (est.step_ms - run["step_ms"]) / run["step_ms"],
                     "breakdown_ms": est.breakdown_ms})
    errs = [r["relative_error"] for r in rows]
    return {"pack": pack.name, "runs": rows,
            "mean_abs_relative_error": sum(abs(e) for e in errs) / len(errs) if errs else None,
            "mean_signed_relative_error": sum(errs) / len(errs) if errs else None}


def fit_coefficient(pack: CalibrationPack, name: str, lo: float, hi: float, iters: int = 40) -> Dict[str, Any]:
    """Value of coefficient ``name`` in ``[lo, hi]`` at which the mean signed error of the pack's runs is
    closest to zero (the prediction is monotone in every coefficient, so bisection applies)."""
    if not pack.observed_runs:
        raise ValueError("the pack has no observed runs to fit to")

    def err(v):
        return evaluate_pack(pack, dict(pack.coefficients, **{name: v}))["mean_signed_relative_error"]
    e_lo, e_hi = err(lo), err(hi)
    if e_lo * e_hi > 0:                              # no sign change: the better end point
        v = lo if abs(e_lo) < abs(e_hi) else hi
    else:
        a, b = lo, hi
        for _ in range(iters):
            m = 0.5 * (a + b)
            if err(m) * e_lo > 0:
                a = m
            else:
                b = m
        v = 0.5 * (a + b)
    return {"coefficient": name, "value": v, "evaluation": evaluate_pack(pack, dict(pack.coefficients, **{name: v}))}
