"""``python -m xorl_b200.sim --model qwen3-8b --gpus 8 --seq-len 4096 [--calibration pack.json]``"""
from __future__ import annotations

import argparse
import json
import os

from ..models.config import ModelConfig, PRESETS, preset
from .planner import HardwareSpec, plan


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default=None, help="preset name or path to a config.json")
    ap.add_argument("--evaluate", action="store_true",
                    help="predicted against observed step times of the calibration pack's runs")
    ap.add_argument("--fit", default=None, metavar="COEF:LO:HI", help="fit one coefficient to the pack's runs")
    ap.add_argument("--list-packs", action="store_true")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--calibration", default=None,
                    help="calibration pack: builtin:<name>, a pack directory, or a JSON of coefficient overrides")
    ap.add_argument("--measured-peaks", default=None, help="JSON with hbm_gbs / bf16_tflops_sustained")
    ap.add_argument("--top", type=int, default=5)
    ns = ap.parse_args(argv)
    from .calibration_packs import evaluate_pack, fit_coefficient, list_calibration_packs, load_pack
    if ns.list_packs:
        print(json.dumps(list_calibration_packs()))
        return list_calibration_packs()
    cal = load_pack(ns.calibration) if ns.calibration else None
    if ns.evaluate or ns.fit:
        if cal is None:
            ap.error("--evaluate / --fit need --calibration")
        if ns.fit:
            name, lo, hi = ns.fit.split(":")
            out = fit_coefficient(cal, name, float(lo), float(hi))
        else:
            out = evaluate_pack(cal)
        print(json.dumps(out, indent=1))
        return out
    if not ns.model:
        ap.error("--model is required")
    cfg = preset(ns.model) if ns.model in PRESETS else ModelConfig.from_pretrained(ns.model)
    hw = HardwareSpec.from_measured(ns.measured_peaks) if ns.measured_peaks and os.path.exists(ns.measured_peaks) \
        else HardwareSpec()
    pack = cal.coefficients if cal is not None else None
    out = [e.to_dict() for e in plan(cfg, ns.gpus, ns.seq_len, hw, pack, ns.top)]
    print(json.dumps(out, indent=1))
    return out


if __name__ == "__main__":
    main()
