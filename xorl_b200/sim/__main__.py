"""``python -m xorl_b200.sim --model qwen3-8b --gpus 8 --seq-len 4096 [--calibration pack.json]``"""
from __future__ import annotations

import argparse
import json
import os

from ..models.config import ModelConfig, PRESETS, preset
from .planner import HardwareSpec, plan


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", required=True, help="preset name or path to a config.json")
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--seq-len", type=int, default=4096)
    ap.add_argument("--calibration", default=None, help="JSON with efficiency overrides")
    ap.add_argument("--measured-peaks", default=None, help="JSON with hbm_gbs / bf16_tflops_sustained")
    ap.add_argument("--top", type=int, default=5)
    ns = ap.parse_args(argv)
    cfg = preset(ns.model) if ns.model in PRESETS else ModelConfig.from_pretrained(ns.model)
    hw = HardwareSpec.from_measured(ns.measured_peaks) if ns.measured_peaks and os.path.exists(ns.measured_peaks) \
        else HardwareSpec()
    pack = json.load(open(ns.calibration)) if ns.calibration else None
    out = [e.to_dict() for e in plan(cfg, ns.gpus, ns.seq_len, hw, pack, ns.top)]
    print(json.dumps(out, indent=1))
    return out


if __name__ == "__main__":
    main()
