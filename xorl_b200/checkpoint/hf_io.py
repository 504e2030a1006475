"""Hugging Face safetensors import / export for models held by the ZeRO engine.

Export gathers one unit at a time (fp32 master -> bf16), splits fused tensors back to HF names and
writes sharded ``model-xxxxx-of-yyyyy.safetensors`` with an index plus ``config.json``
(src/xorl/models/module_utils.py:2594-2825).  Import streams the safetensors files and fills each
rank's shard (src/xorl/models/module_utils.py:1337-1917)."""
from __future__ import annotations

import json
import os
from typing import Dict, List

import torch
import torch.distributed as dist

from .handlers import get_checkpoint_handler


def save_hf_weights(engine, out_dir: str, cfg, dtype: torch.dtype = torch.bfloat16,
                    max_shard_bytes: int = 5 * 2 ** 30) -> None:
    from safetensors.torch import save_file
    rank0 = engine.ps.rank == 0
    handler = get_checkpoint_handler(cfg)
    if rank0:
        os.makedirs(out_dir, exist_ok=True)
    shards: List[Dict[str, torch.Tensor]] = [{}]
    size = 0
    tied = cfg.tie_word_embeddings
    for name, full in engine.iter_full_tensors("master"):
        if not rank0:
            continue
        for hf_name, t in handler.to_hf(name, full):
            t = t.to(dtype).cpu().contiguous()
            nbytes = t.numel() * t.element_size()
            if size + nbytes > max_shard_bytes and shards[-1]:
                shards.append({})
                size = 0
            shards[-1][hf_name] = t
            size += nbytes
    if rank0:
        n = len(shards)
        weight_map = {}
        for i, sd in enumerate(shards):
            fname = "model.safetensors" if n == 1 else f"model-{i + 1:05d}-of-{n:05d}.safetensors"
            save_file(sd, os.path.join(out_dir, fname), metadata={"format": "pt"})
            for k in sd:
                weight_map[k] = fname
        if n > 1:
            with open(os.path.join(out_dir, "model.safetensors.index.json"), "w") as f:
                json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=2)
        cfg.save_pretrained(out_dir)
    if dist.is_initialized():
        dist.barrier()


def _open_index(path: str) -> Dict[str, str]:
    idx = os.path.join(path, "model.safetensors.index.json")
    if os.path.exists(idx):
        with open(idx) as f:
            return json.load(f)["weight_map"]
    from safetensors import safe_open
    out = {}
    for fn in sorted(os.listdir(path)):
        if fn.endswith(".safetensors"):
            with safe_open(os.path.join(path, fn), "pt") as f:
                for k in f.keys():
                    out[k] = fn
    return out


def load_hf_weights(engine, path: str, cfg, strict: bool = True) -> List[str]:
    """Every rank reads the tensors it needs (all ranks read; the page cache serves repeats)."""
    from safetensors import safe_open
    handler = get_checkpoint_handler(cfg)
    weight_map = _open_index(path)
    handles: Dict[str, object] = {}

    def read(name: str) -> torch.Tensor:
        fn = weight_map[name]
        if fn not in handles:
            handles[fn] = safe_open(os.path.join(path, fn), "pt")
        return handles[fn].get_tensor(name)

    missing: List[str] = []
    for g in engine.all_groups():
        tensors = {}
        for i, _, _ in g.param_segments_in_shard():
            pname = g.named_params[i][0]
            srcs = handler.hf_sources(pname)
            if cfg.tie_word_embeddings and pname.startswith("lm_head"):
                srcs = ["model.embed_tokens.weight"]
            if not all(s in weight_map for s in srcs):
                missing.append(pname)
                continue
            tensors[pname] = handler.from_hf(pname, [read(s) for s in srcs])
        engine.load_full_tensors(tensors, strict=False) if tensors else None
    if strict and missing:
        raise KeyError(f"weights missing from {path}: {missing[:8]}")
    return missing
