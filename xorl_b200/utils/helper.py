"""Seeding, EnvironMeter (tokens/s, MFU, memory), CUDA-event timers, torch-profiler factory.

EnvironMeter reports the same metric names as the reference (src/xorl/utils/helper.py:80-198):
``efficiency/mfu``, ``flops_achieved(T)``, ``tokens_per_second(K)``, ``consume_tokens(B)``,
``memory/*``.  Step time may come from the host clock (reference definition) or from CUDA events.
"""
from __future__ import annotations

import os
import random
import time
from contextlib import contextmanager
from typing import Any, Dict, List, Optional

import numpy as np
import torch
import torch.distributed as dist

from .count_flops import get_device_flops, model_flops_per_token


def set_seed(seed: int, full_determinism: bool = False) -> None:
    random.seed(seed)
    np.random.seed(seed % (2 ** 32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    if full_determinism:
        os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":4096:8")
        torch.use_deterministic_algorithms(True, warn_only=True)


class EnvironMeter:
    def __init__(self, config, world_size: int = 1, dp_group=None, recompute: bool = True):
        self.config = config
        self.world_size = world_size
        self.dp_group = dp_group
        self.recompute = recompute
        self.consumed_tokens = 0
        self.batch_tokens = 0
        self.batch_lens: List[int] = []
        self.peak = get_device_flops() if torch.cuda.is_available() else 1e12

    def add(self, micro_batch: Dict[str, torch.Tensor]) -> None:
        cu = micro_batch.get("cu_seqlens")
        if cu is not None and not cu.is_cuda:
            c = cu.tolist()
            self.batch_lens += [b - a for a, b in zip(c[:-1], c[1:])]
        self.batch_tokens += int(micro_batch["input_ids"].numel())

    def step(self, delta_time: float, global_step: int = 0) -> Dict[str, float]:
        tokens = torch.tensor([float(self.batch_tokens),
                               float(self.batch_tokens) * model_flops_per_token(
                                   self.config, self.batch_lens or None, True, self.recompute)],
                              dtype=torch.float64)
        if dist.is_initialized() and self.world_size > 1:
            t = tokens.to("cuda" if torch.cuda.is_available() and dist.get_backend() == "nccl" else "cpu")
            dist.all_reduce(t)
            tokens = t.cpu()
        tok, flops = float(tokens[0]), float(tokens[1])
        self.consumed_tokens += int(tok)
        out = {
            "efficiency/mfu": flops / max(delta_time, 1e-9) / (self.peak * self.world_size),
            "flops_achieved(T)": flops / max(delta_time, 1e-9) / 1e12 / self.world_size,
            "tokens_per_second(K)": tok / max(delta_time, 1e-9) / 1e3,
            "consume_tokens(B)": self.consumed_tokens / 1e9,
        }
        if torch.cuda.is_available():
            out["memory/max_allocated(GB)"] = torch.cuda.max_memory_allocated() / 2 ** 30
            out["memory/max_reserved(GB)"] = torch.cuda.max_memory_reserved() / 2 ** 30
        self.batch_tokens, self.batch_lens = 0, []
        return out

    def state_dict(self):
        return {"consumed_tokens": self.consumed_tokens}

    def load_state_dict(self, sd):
        self.consumed_tokens = int(sd.get("consumed_tokens", 0))


class CudaTimer:
    """CUDA-event scoped timers (cf. src/xorl/utils/manual_cuda_timing.py)."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled and torch.cuda.is_available()
        self.records: Dict[str, List] = {}

    @contextmanager
    def scope(self, name: str):
        if not self.enabled:
            t0 = time.perf_counter()
            yield
            self.records.setdefault(name, []).append(("host", (time.perf_counter() - t0) * 1e3))
            return
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self.records.setdefault(name, []).append(("cuda", a, b))

    def summary(self) -> Dict[str, float]:
        if self.enabled:
            torch.cuda.synchronize()
        out = {}
        for k, rs in self.records.items():
            ms = [r[1] if r[0] == "host" else r[1].elapsed_time(r[2]) for r in rs]
            out[k] = sum(ms)
        self.records = {}
        return out


def create_profiler(start_step: int, end_step: int, trace_dir: str, record_shapes: bool = True,
                    profile_memory: bool = True, with_stack: bool = True, rank: int = 0):
    """torch.profiler with a wait/warmup/active schedule writing
    ``xorl_rank{r}_{ts}.pt.trace.json.gz`` (src/xorl/utils/helper.py:506-576)."""
    from torch.profiler import ProfilerActivity, profile, schedule
    os.makedirs(trace_dir, exist_ok=True)

    def handler(prof):
        path = os.path.join(trace_dir, f"xorl_rank{rank}_{int(time.time())}.pt.trace.json.gz")
        prof.export_chrome_trace(path)

    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
    return profile(activities=acts,
                   schedule=schedule(wait=max(0, start_step - 1), warmup=1 if start_step > 0 else 0,
                                     active=max(1, end_step - start_step), repeat=1),
                   on_trace_ready=handler, record_shapes=record_shapes,
                   profile_memory=profile_memory, with_stack=with_stack)
