"""Write a quantised Hugging Face checkpoint from a bf16/fp32 one.

    python -m xorl_b200.cli.export_quantized --src <hf_dir> --dst <out_dir> --format block_fp8|nvfp4|mxfp4|nf4|int4
        [--group-size N] [--skip lm_head embed_tokens norm gate]

Streams tensor by tensor (a shard of the source is mapped at a time, the output is written in
shards of ``--shard-gb``), quantises every 2-D weight whose name matches none of ``--skip`` and
stores the packed codes under the original name with companion scale tensors
(``<name>_scale_inv`` for block-fp8, ``<name>_scale`` / ``<name>_scale_2`` for nvfp4, ``<name>_scale``
otherwise), plus a ``quantization_config`` block in ``config.json``
(src/xorl/cli/export_quantized.py)."""
from __future__ import annotations

import argparse
import json
import os
import shutil
from typing import Dict, Iterator, List, Optional, Tuple

import torch

from ..ops import quantize as Q

DEFAULT_SKIP = ("lm_head", "embed_tokens", "norm", ".gate.", "router", "bias", "sinks")
DEFAULT_GROUP = {"block_fp8": 128, "nvfp4": 16, "mxfp4": 32, "nf4": 64, "int4": 128}


def iter_hf_tensors(src: str) -> Iterator[Tuple[str, torch.Tensor]]:
    from safetensors import safe_open
    files = sorted(f for f in os.listdir(src) if f.endswith(".safetensors"))
    if not files:
        raise FileNotFoundError(f"no .safetensors files in {src}")
    for f in files:
        with safe_open(os.path.join(src, f), "pt") as fh:
            for k in fh.keys():
                yield k, fh.get_tensor(k)


def quantize_entry(name: str, t: torch.Tensor, fmt: str, group: int, skip=DEFAULT_SKIP) -> Dict[str, torch.Tensor]:
    if t.dim() != 2 or any(s in name for s in skip) or not name.endswith("weight"):
        return {name: t}
    if fmt == "block_fp8":
        q, s = Q.block_fp8_quantize_128x128(t.float())
        return {name: q, name + "_scale_inv": s}
    if t.shape[-1] % group:
        return {name: t}
    if fmt == "nvfp4":
        packed, bs, gs = Q.nvfp4_quantize(t.float(), group)
        return {name: packed, name + "_scale": bs, name + "_scale_2": gs.reshape(1).float()}
    parts = Q.quantize_weight(t.float(), fmt, group)
    out = {name: parts["packed"], name + "_scale": parts["scale"]}
    out[name + "_shape"] = torch.tensor(list(t.shape), dtype=torch.int64)
    return out


def export(src: str, dst: str, fmt: str, group: Optional[int] = None, skip=DEFAULT_SKIP,
           shard_gb: float = 4.0) -> Dict[str, int]:
    from safetensors.torch import save_file
    group = group or DEFAULT_GROUP[fmt]
    os.makedirs(dst, exist_ok=True)
    weight_map: Dict[str, str] = {}
    pending: Dict[str, torch.Tensor] = {}
    size, shard, stats = 0, 0, {"quantized": 0, "kept": 0, "bytes_in": 0, "bytes_out": 0}

    def flush():
        nonlocal pending, size, shard
        if not pending:
            return
        shard += 1
        fname = f"model-{shard:05d}.safetensors"
        save_file({k: v.contiguous() for k, v in pending.items()}, os.path.join(dst, fname))
        for k in pending:
            weight_map[k] = fname
        pending, size = {}, 0

    for name, t in iter_hf_tensors(src):
        out = quantize_entry(name, t, fmt, group, skip)
        stats["quantized" if len(out) > 1 else "kept"] += 1
        stats["bytes_in"] += t.numel() * t.element_size()
        for k, v in out.items():
            pending[k] = v
            nb = v.numel() * v.element_size()
            size += nb
            stats["bytes_out"] += nb
        if size >= shard_gb * (1 << 30):
            flush()
    flush()
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": stats["bytes_out"]}, "weight_map": weight_map}, f, indent=1)
    for aux in os.listdir(src):
        if aux.endswith((".json", ".txt", ".model", ".jinja")) and aux != "model.safetensors.index.json":
            shutil.copy(os.path.join(src, aux), os.path.join(dst, aux))
    cfg_path = os.path.join(dst, "config.json")
    cfg = {}
    if os.path.exists(cfg_path):
        with open(cfg_path) as f:
            cfg = json.load(f)
    qc = {"quant_method": {"block_fp8": "fp8", "nvfp4": "modelopt_fp4"}.get(fmt, fmt), "format": fmt,
          "group_size": group, "ignore": list(skip)}
    if fmt == "block_fp8":
        qc.update(fmt="e4m3", activation_scheme="dynamic", weight_block_size=[128, 128])
    cfg["quantization_config"] = qc
    with open(cfg_path, "w") as f:
        json.dump(cfg, f, indent=2)
    return stats


def main(argv: Optional[List[str]] = None, default_format: Optional[str] = None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--src", required=True)
    ap.add_argument("--dst", required=True)
    ap.add_argument("--format", default=default_format or "block_fp8", choices=sorted(DEFAULT_GROUP))
    ap.add_argument("--group-size", type=int, default=None)
    ap.add_argument("--skip", nargs="*", default=list(DEFAULT_SKIP))
    ap.add_argument("--shard-gb", type=float, default=4.0)
    ns = ap.parse_args(argv)
    stats = export(ns.src, ns.dst, ns.format, ns.group_size, tuple(ns.skip), ns.shard_gb)
    print(json.dumps(stats))
    return stats


if __name__ == "__main__":
    main()
