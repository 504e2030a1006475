"""``python -m xorl_b200.cli.export_nvfp4 --src <hf_dir> --dst <out_dir>``: a servable NVFP4 checkpoint from
a bf16 Hugging Face one (for instance the master weights saved by a fake-quantised RL run)
(src/xorl/cli/export_nvfp4.py).

Per quantised ``<name>.weight [out, in]``:

* ``<name>.weight``          uint8 ``[out, in / 2]``, two e2m1 codes per byte (even column in the low nibble);
* ``<name>.weight_scale``    e4m3  ``[out, in / 16]``, one scale per group of 16 along ``in``;
* ``<name>.weight_scale_2``  fp32 scalar, the per-tensor scale;
* ``<name>.input_scale``     fp32 scalar, only with ``--act-amax``: the activation scale a W4A4 server needs,

plus ``hf_quant_config.json`` (``quant_algo: NVFP4``) and a ``quantization_config`` block in ``config.json``.
Projections that inference engines fuse into one GEMM (q / k / v and gate / up of one layer) must share one
``weight_scale_2``, or the fused kernel mis-scales all members but one: a first pass over the tensor headers
and the members' maxima finds the shared scale of every such group.  The rounding is the one the fake-quant
training path uses (``ops.quantize.nvfp4_quantize``), so the exported values are the ones trained against."""
from __future__ import annotations

import argparse
import fnmatch
import json
import os
import shutil
from typing import Dict, List, Optional

import torch

from ..ops import quantize as Q

KEEP = ("*lm_head*", "*embed_tokens*", "*norm*", "*mlp.gate.weight", "*.gate.weight", "*router*", "*sinks*")
FUSED = {"q_proj": "qkv", "k_proj": "qkv", "v_proj": "qkv", "gate_proj": "gate_up", "up_proj": "gate_up"}
E2M1_MAX = 6.0


def fused_group(module: str) -> Optional[str]:
    """``...self_attn.q_proj`` -> ``...self_attn::qkv``; None for a projection that stands alone."""
    parent, _, short = module.rpartition(".")
    return f"{parent}::{FUSED[short]}" if short in FUSED else None


def _kept(name: str, keep) -> bool:
    return any(fnmatch.fnmatch(name, p) for p in keep)


def _size_bytes(text: Optional[str], default: int) -> int:
    if not text:
        return default
    t = text.strip().upper()
    for suffix, mult in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10), ("B", 1)):
        if t.endswith(suffix):
            return int(float(t[: -len(suffix)]) * mult)
    return int(t)


def quantize_weight(w: torch.Tensor, group: int = 16, global_scale: Optional[torch.Tensor] = None,
                    act_amax: float = 0.0) -> Dict[str, torch.Tensor]:
    out_f, in_f = w.shape
    packed, bs, gs = Q.nvfp4_quantize(w.float().contiguous(), group, global_scale=global_scale)
    entry = {"weight": packed.reshape(out_f, in_f // 2), "weight_scale": bs.reshape(out_f, in_f // group),
             "weight_scale_2": gs.reshape(()).float().clone()}
    if act_amax > 0:
        entry["input_scale"] = torch.tensor(act_amax / (E2M1_MAX * Q.FP8_MAX), dtype=torch.float32)
    return entry


def export(src: str, dst: str, group: int = 16, keep=KEEP, max_shard_bytes: int = 5 << 30,
           overwrite: bool = False, act_amax: Optional[Dict[str, float]] = None) -> Dict[str, int]:
    from safetensors import safe_open
    from safetensors.torch import save_file
    if group != 16:
        raise ValueError("nvfp4 groups are 16 wide: serving kernels assume it")
    if os.path.isdir(dst) and os.listdir(dst) and not overwrite:
        raise FileExistsError(f"{dst} is not empty (pass --overwrite)")
    cfg = {}
    if os.path.exists(os.path.join(src, "config.json")):
        with open(os.path.join(src, "config.json")) as f:
            cfg = json.load(f)
    for k in ("num_nextn_predict_layers", "mtp_num_hidden_layers", "mtp_num_layers"):
        if isinstance(cfg.get(k), int) and cfg[k] > 0:
            raise ValueError(f"checkpoints with multi-token-prediction layers ({k}={cfg[k]}) are not exported")
    files = sorted(f for f in os.listdir(src) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {src}")

    def convertible(name, shape) -> bool:
        return name.endswith(".weight") and len(shape) == 2 and shape[1] % group == 0 and not _kept(name, keep)

    # pass 1: the shared maximum of every fused group
    group_amax: Dict[str, torch.Tensor] = {}
    for fn in files:
        with safe_open(os.path.join(src, fn), "pt") as fh:
            for name in fh.keys():
                g = fused_group(name[: -len(".weight")]) if name.endswith(".weight") else None
                if g is None or not convertible(name, fh.get_slice(name).get_shape()):
                    continue
                amax = fh.get_tensor(name).float().abs().max()
                group_amax[g] = torch.maximum(group_amax[g], amax) if g in group_amax else amax
    os.makedirs(dst, exist_ok=True)
    weight_map: Dict[str, str] = {}
    pending: Dict[str, torch.Tensor] = {}
    stats = {"quantized": 0, "kept": 0, "bytes_in": 0, "bytes_out": 0, "fused_groups": len(group_amax)}
    size, shard, excluded = 0, 0, []

    def flush():
        nonlocal pending, size, shard
        if pending:
            shard += 1
            fname = f"model-{shard:05d}.safetensors"
            save_file({k: v.contiguous() for k, v in pending.items()}, os.path.join(dst, fname))
            weight_map.update({k: fname for k in pending})
            pending, size = {}, 0

    # pass 2: quantise and write
    for fn in files:
        with safe_open(os.path.join(src, fn), "pt") as fh:
            for name in fh.keys():
                t = fh.get_tensor(name)
                stats["bytes_in"] += t.numel() * t.element_size()
                if convertible(name, t.shape):
                    mod = name[: -len(".weight")]
                    g = fused_group(mod)
                    gs = (group_amax[g].clamp_min(1e-12) / (E2M1_MAX * Q.FP8_MAX)) if g in group_amax else None
                    out = {f"{mod}.{k}": v for k, v in quantize_weight(t, group, gs, float((act_amax or {}).get(mod, 0.0))).items()}
                    stats["quantized"] += 1
                else:
                    out = {name: t}
                    stats["kept"] += 1
                    if name.endswith(".weight") and t.dim() == 2:
                        excluded.append(name[: -len(".weight")])
                for k, v in out.items():
                    pending[k] = v
                    nb = v.numel() * v.element_size()
                    size += nb
                    stats["bytes_out"] += nb
                if size >= max_shard_bytes:
                    flush()
    flush()
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": stats["bytes_out"]}, "weight_map": weight_map}, f, indent=1)
    for aux in os.listdir(src):
        if aux.endswith((".json", ".txt", ".model", ".jinja")) and aux not in ("model.safetensors.index.json", "config.json"):
            shutil.copy(os.path.join(src, aux), os.path.join(dst, aux))
    quant = {"quant_algo": "NVFP4", "kv_cache_quant_algo": None, "group_size": group, "exclude_modules": sorted(set(excluded))}
    with open(os.path.join(dst, "hf_quant_config.json"), "w") as f:
        json.dump({"producer": {"name": "xorl_b200"}, "quantization": quant}, f, indent=2)
    cfg["quantization_config"] = {"quant_method": "modelopt_fp4", "format": "nvfp4", **quant,
                                  "activation": bool(act_amax)}
    with open(os.path.join(dst, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return stats


def main(argv: Optional[List[str]] = None):
    ap = argparse.ArgumentParser(description="bf16 Hugging Face checkpoint -> servable NVFP4 checkpoint")
    ap.add_argument("--src", "--input-dir", dest="src", required=True)
    ap.add_argument("--dst", "--output-dir", dest="dst", required=True)
    ap.add_argument("--group-size", type=int, default=16)
    ap.add_argument("--max-shard-size", default=None, help="e.g. 5GB")
    ap.add_argument("--overwrite", action="store_true")
    ap.add_argument("--modules-to-not-convert", nargs="*", default=None,
                    help="glob patterns on the full tensor name (default: lm-head, embeddings, norms, routers)")
    ap.add_argument("--act-amax", default=None,
                    help="JSON file {module: activation amax} (or a calibration summary with 'modules': "
                         "{name: {'input_amax': ...}}); adds input_scale for W4A4 serving")
    ns = ap.parse_args(argv)
    amax = None
    if ns.act_amax:
        with open(ns.act_amax) as f:
            raw = json.load(f)
        raw = raw.get("modules", raw)
        amax = {k: float(v["input_amax"] if isinstance(v, dict) else v) for k, v in raw.items()
                if (v.get("input_amax") if isinstance(v, dict) else v)}
    stats = export(ns.src, ns.dst, ns.group_size, tuple(ns.modules_to_not_convert or KEEP),
                   _size_bytes(ns.max_shard_size, 5 << 30), ns.overwrite, amax)
    print(json.dumps(stats))
    return stats


if __name__ == "__main__":
    main()
