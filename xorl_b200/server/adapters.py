"""Many named LoRA adapters over one frozen base model.

The engine holds exactly one *active* adapter in its trainable flat shards (with LoRA enabled the
trainable parameter groups are the adapter matrices and nothing else).  Inactive adapters live in
pinned host memory as per-group snapshots of the fp32 master shard, the accumulated gradient and
every optimizer state tensor, together with their step counters and open gradient epoch.  Switching
is two shard-sized copies per group; the least recently used adapter is evicted (to disk when a
directory is given) once ``XORL_MAX_ADAPTERS_PER_MODEL`` snapshots exist
(src/xorl/server/runner/adapters/manager.py, sharded_state.py).  Every rank runs the same sequence
of calls, so shards stay consistent without communication."""
from __future__ import annotations

import os
from collections import OrderedDict
from typing import Any, Dict, List, Optional

import torch


class AdapterState:
    def __init__(self):
        self.groups: List[Dict[str, torch.Tensor]] = []
        self.meta: Dict[str, Any] = {}


class AdapterManager:
    def __init__(self, runner, max_adapters: Optional[int] = None, spill_dir: Optional[str] = None):
        self.runner = runner
        self.engine, self.optimizer = runner.engine, runner.optimizer
        self.max_adapters = max_adapters or int(os.environ.get("XORL_MAX_ADAPTERS_PER_MODEL", "8"))
        self.spill_dir = spill_dir
        self.active: str = "default"
        self.store: "OrderedDict[str, AdapterState]" = OrderedDict()
        self.known = {"default"}
        self._groups = [g for g in self.engine.all_groups() if not getattr(g, "frozen", False)]
        if not self._groups:
            raise RuntimeError("no trainable parameter groups")
        self._pristine = self._snapshot()           # freshly initialised adapter (B = 0): template for new ones
        self._pristine.meta = {"step": 0, "opt_step": 0, "epoch_open": False, "tokens": 0}

    # ---- snapshots --------------------------------------------------------------------------
    def _host(self, t: torch.Tensor) -> torch.Tensor:
        h = torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=t.is_cuda)
        h.copy_(t, non_blocking=t.is_cuda)
        return h

    def _snapshot(self) -> AdapterState:
        st = AdapterState()
        self.engine.sync_optimizer()             # shards are read outside the step path
        for g in self._groups:
            d = {"master": self._host(g.master), "grad": self._host(g.grad_shard)}
            for name, per_group in self.optimizer.state.items():
                if id(g) in per_group:
                    d["opt." + name] = self._host(per_group[id(g)])
            d["grad_ready"] = torch.tensor(int(g.grad_ready))
            st.groups.append(d)
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        r = self.runner
        st.meta = {"step": r.step, "opt_step": self.optimizer.step_count, "epoch_open": r.epoch_open,
                   "tokens": r.accumulated_tokens}
        return st

    def _restore(self, st: AdapterState) -> None:
        self.engine.sync_optimizer()
        for g, d in zip(self._groups, st.groups):
            g.master.copy_(d["master"], non_blocking=True)
            g.grad_shard.copy_(d["grad"], non_blocking=True)
            g.grad_ready = bool(int(d["grad_ready"]))
            for name, per_group in self.optimizer.state.items():
                if "opt." + name in d:
                    per_group[id(g)].copy_(d["opt." + name], non_blocking=True)
            self.engine.refresh_compute_copy(g)
        r = self.runner
        r.step, r.epoch_open, r.accumulated_tokens = st.meta["step"], st.meta["epoch_open"], st.meta["tokens"]
        self.optimizer.step_count = st.meta["opt_step"]

    # ---- public ------------------------------------------------------------------------------
    def create(self, model_id: str) -> None:
        if model_id in self.known:
            raise ValueError(f"adapter {model_id!r} exists")
        self.known.add(model_id)
        fresh = AdapterState()
        fresh.groups = [{k: v.clone() for k, v in d.items()} for d in self._pristine.groups]
        fresh.meta = dict(self._pristine.meta)
        self._put(model_id, fresh)

    def _put(self, model_id: str, st: AdapterState) -> None:
        self.store[model_id] = st
        self.store.move_to_end(model_id)
        while len(self.store) > self.max_adapters - 1:          # one more lives in the engine
            victim, vst = self.store.popitem(last=False)
            if self.spill_dir:
                os.makedirs(self.spill_dir, exist_ok=True)
                torch.save({"groups": vst.groups, "meta": vst.meta}, self._spill_path(victim))
            else:
                self.known.discard(victim)

    def _spill_path(self, model_id: str) -> str:
        rank = self.engine.ps.rank
        return os.path.join(self.spill_dir, f"{model_id}.rank{rank}.pt")

    def activate(self, model_id: str) -> None:
        if model_id == self.active:
            return
        if model_id not in self.known:
            raise KeyError(f"unknown adapter {model_id!r}")
        st = self.store.pop(model_id, None)
        if st is None:
            if not (self.spill_dir and os.path.exists(self._spill_path(model_id))):
                raise KeyError(f"adapter {model_id!r} was evicted")
            blob = torch.load(self._spill_path(model_id), weights_only=False)
            st = AdapterState()
            st.groups, st.meta = blob["groups"], blob["meta"]
        current = self._snapshot()
        self._restore(st)
        self._put(self.active, current)
        self.active = model_id

    def unload(self, model_id: str) -> None:
        if model_id == "default":
            return
        if model_id == self.active:
            self.activate("default")
        self.store.pop(model_id, None)
        self.known.discard(model_id)
        if self.spill_dir and os.path.exists(self._spill_path(model_id)):
            os.remove(self._spill_path(model_id))

    def list(self) -> List[str]:
        return sorted(self.known)
