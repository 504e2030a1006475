"""Expert-load metrics of MoE layers.

The router's per-expert token counts of every MoE layer are accumulated on the device while the
model runs (no host synchronisation); ``collect`` sums them over the data-parallel group, reads them
once and reports, per layer and over all layers, the most and least loaded expert and the imbalance
ratio (max load / mean load), plus allocator statistics, as one JSON line per step in
``moe_metrics.jsonl`` on rank 0 (src/xorl/server/runner/utils/moe_metrics.py:30-175).
"""
from __future__ import annotations

import json
import os
import time
from typing import Any, Dict, Optional

import torch
import torch.distributed as dist


class ExpertLoadTracker:
    def __init__(self, num_experts: int, output_dir: Optional[str] = None, rank: int = 0, group=None,
                 per_layer_detail: int = 2):
        self.num_experts = int(num_experts or 0)
        self.enabled = self.num_experts > 0
        self.rank, self.group = rank, group
        self.loads: Dict[int, torch.Tensor] = {}
        self.per_layer_detail = per_layer_detail
        self.path = os.path.join(output_dir, "moe_metrics.jsonl") if (output_dir and self.enabled) else None
        if self.path and rank == 0:
            os.makedirs(output_dir, exist_ok=True)

    # called by the engine after every first-pass layer forward
    def add(self, layer_idx: int, counts: torch.Tensor) -> None:
        if not self.enabled:
            return
        cur = self.loads.get(layer_idx)
        self.loads[layer_idx] = counts.detach().to(torch.int64).clone() if cur is None else cur.add_(counts)

    def reset(self) -> None:
        self.loads.clear()

    def collect(self, step: int, seconds: float = 0.0) -> Dict[str, Any]:
        out: Dict[str, Any] = {"step": int(step), "forward_backward_time": float(seconds), "timestamp": time.time()}
        if self.enabled and self.loads:
            layers = sorted(self.loads)
            stacked = torch.stack([self.loads[l] for l in layers])                     # [L, E]
            if self.group is not None and dist.is_initialized() and dist.get_world_size(self.group) > 1:
                dist.all_reduce(stacked, group=self.group)
            host = stacked.cpu().double()
            total = host.sum(1)
            mean = (total / self.num_experts).clamp_min(1e-9)
            mx, mn = host.max(1).values, host.min(1).values
            imb = mx / mean
            per_layer = {f"layer_{l}": {"max_load": int(mx[i]), "min_load": int(mn[i]), "total_tokens": int(total[i]),
                                        "imbalance_ratio": float(imb[i]), "idle_experts": int((host[i] == 0).sum())}
                         for i, l in enumerate(layers)}
            keep = set(layers[:self.per_layer_detail] + layers[-self.per_layer_detail:])
            out["expert_load"] = {
                "num_moe_layers": len(layers), "total_tokens": int(total.sum()),
                "mean_imbalance_ratio": float(imb.mean()), "max_imbalance_ratio": float(imb.max()),
                "mean_max_load": float(mx.mean()), "mean_min_load": float(mn.mean()),
                "per_layer": {k: v for k, v in per_layer.items() if int(k.split("_")[1]) in keep}}
        if torch.cuda.is_available():
            stats = torch.cuda.memory_stats()
            out["memory"] = {"allocated_gb": torch.cuda.memory_allocated() / 1e9,
                             "reserved_gb": torch.cuda.memory_reserved() / 1e9,
                             "max_allocated_gb": torch.cuda.max_memory_allocated() / 1e9,
                             "num_alloc_retries": stats.get("num_alloc_retries", 0), "num_ooms": stats.get("num_ooms", 0)}
        self.reset()
        return out

    def write(self, metrics: Dict[str, Any]) -> None:
        if self.rank != 0 or self.path is None:
            return
        with open(self.path, "a") as f:
            f.write(json.dumps(metrics, separators=(",", ":")) + "\n")
