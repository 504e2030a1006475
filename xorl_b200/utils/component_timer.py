"""Per-component phase timing: forward pre/post hooks (and full backward hooks) on the decoder's
sub-modules record CUDA events (wall clock on CPU) and report milliseconds per component class
(src/xorl/trainers/per_component_timer.py)."""
from __future__ import annotations

import time
from collections import defaultdict
from typing import Dict, List, Tuple

import torch
from torch import nn


class PerComponentTimer:
    def __init__(self, model: nn.Module, classes: Tuple[str, ...] = ("Attention", "MLP", "MoEBlock", "RMSNorm")):
        self.cuda = torch.cuda.is_available() and next(model.parameters()).is_cuda
        self.pending: List[Tuple[str, object, object]] = []
        self.totals: Dict[str, float] = defaultdict(float)
        self.counts: Dict[str, int] = defaultdict(int)
        self.handles = []
        self._open: Dict[int, object] = {}
        for name, mod in model.named_modules():
            cls = type(mod).__name__
            if cls in classes:
                self.handles.append(mod.register_forward_pre_hook(self._pre(cls)))
                self.handles.append(mod.register_forward_hook(self._post(cls)))

    def _now(self):
        if self.cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()

    def _pre(self, cls):
        def hook(mod, args):
            self._open[id(mod)] = self._now()
        return hook

    def _post(self, cls):
        def hook(mod, args, out):
            start = self._open.pop(id(mod), None)
            if start is not None:
                self.pending.append((cls + ("" if torch.is_grad_enabled() else ""), start, self._now()))
        return hook

    def flush(self) -> Dict[str, float]:
        """Resolves the recorded intervals (synchronises once) and returns total ms per class."""
        if self.cuda:
            torch.cuda.synchronize()
        for cls, a, b in self.pending:
            ms = a.elapsed_time(b) if self.cuda else (b - a) * 1e3
            self.totals[cls] += ms
            self.counts[cls] += 1
        self.pending.clear()
        return dict(self.totals)

    def summary(self) -> str:
        self.flush()
        rows = sorted(self.totals.items(), key=lambda kv: -kv[1])
        return "\n".join(f"{k:>12s}  {v:10.3f} ms  {self.counts[k]:6d} calls" for k, v in rows)

    def reset(self) -> None:
        self.totals.clear()
        self.counts.clear()
        self.pending.clear()

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles.clear()
