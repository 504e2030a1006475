"""Many named LoRA adapters over one frozen base model.

The engine holds exactly one *active* adapter in its trainable flat shards (with LoRA enabled the
trainable parameter groups are the adapter matrices and nothing else).  Inactive adapters live in
pinned host memory as per-group snapshots of the fp32 master shard, the accumulated gradient and
every optimizer state tensor, together with their step counters and open gradient epoch.  Switching
is two shard-sized copies per group; the least recently used adapter is evicted (to disk when a
directory is given) once ``XORL_MAX_ADAPTERS_PER_MODEL`` snapshots exist
(src/xorl/server/runner/adapters/manager.py, sharded_state.py).  Every rank runs the same sequence
of calls, so shards stay consistent without communication.

A session may ask for a lower rank than the model's adapter capacity ``R`` and for its own alpha
(``create(model_id, {"rank": r, "alpha": a})``): its A rows and B columns from ``r`` up start at zero,
and a rank component whose A row and B column are both zero has zero gradient in both, so it stays zero
under any of the optimizers -- the adapter is exactly a rank-``r`` adapter in rank-``R`` storage, scaled
by ``a / r``.  The learning rate last used by a session stays with it.  An adapter that holds
accumulated gradients is never dropped: eviction takes the least recently used adapter without an open
gradient epoch, or writes the victim to the spill directory with its gradients."""
from __future__ import annotations

import math
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
        from ..adapters.lora import ExpertsLoRA, LoraLinear
        self._lora_modules = [m for m in self.engine.model.modules() if isinstance(m, (LoraLinear, ExpertsLoRA))]
        if not self._lora_modules:
            raise RuntimeError("the model carries no LoRA modules")
        self.capacity = int(self._lora_modules[0].rank)
        self.default_alpha = float(self._lora_modules[0].scaling) * self.capacity
        self._pristine = self._snapshot()           # freshly initialised adapter (B = 0): template for new ones
        self._pristine.meta = {"step": 0, "opt_step": 0, "epoch_open": False, "tokens": 0,
                               "scaling": float(self._lora_modules[0].scaling), "lr": float(self.optimizer.lr),
                               "rank": self.capacity, "alpha": self.default_alpha}
        self.session = dict(rank=self.capacity, alpha=self.default_alpha)     # of the active adapter

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
                   "tokens": r.accumulated_tokens, "scaling": float(self._lora_modules[0].scaling),
                   "lr": float(self.optimizer.lr), **getattr(self, "session", {})}
        return st

    def _rank_index(self, p: torch.nn.Parameter, shape, idx: torch.Tensor) -> Optional[torch.Tensor]:
        """Rank component of flat element ``idx`` of adapter matrix ``p`` (None: not an adapter matrix).
        Dense: A [R, in], B [out, R]; experts: A [E, in, R], B [E, R, out]."""
        kind = getattr(p, "_xb_lora", None)
        if kind is None:
            return None
        kind = "B" if kind.startswith("B") else kind
        shape = tuple(shape)
        if len(shape) == 2:
            return idx // shape[1] if kind == "A" else idx % shape[1]
        return idx % shape[2] if kind == "A" else (idx // shape[2]) % shape[1]

    def _truncate_rank(self, st: AdapterState, rank: int) -> None:
        """Zeroes the rank components from ``rank`` up in the master shards of a fresh snapshot."""
        for g, d in zip(self._groups, st.groups):
            lo, hi = g.rank * g.shard_numel, (g.rank + 1) * g.shard_numel
            for (name, p), off, shape in zip(g.named_params, g.offsets, g.shapes):
                a, b = max(lo, off), min(hi, off + math.prod(shape))
                if a >= b:
                    continue
                comp = self._rank_index(p, shape, torch.arange(a - off, b - off))
                if comp is None:
                    continue
                view = d["master"][a - lo:b - lo]
                view[comp >= rank] = 0

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
        if "scaling" in st.meta:
            for m in self._lora_modules:
                m.scaling = st.meta["scaling"]
        if "lr" in st.meta:
            self.optimizer.set_lr(float(st.meta["lr"]))
        self.session = dict(rank=st.meta.get("rank", self.capacity), alpha=st.meta.get("alpha", self.default_alpha))

    # ---- public ------------------------------------------------------------------------------
    def create(self, model_id: str, lora_config: Optional[Dict[str, Any]] = None) -> None:
        """``lora_config``: ``rank`` (<= the model's adapter capacity), ``alpha``, ``learning_rate``
        (src/xorl/server/runner/adapters/manager.py:1911-1920,2181-2320)."""
        if model_id in self.known:
            raise ValueError(f"adapter {model_id!r} exists")
        cfg = dict(lora_config or {})
        rank = int(cfg.get("rank", cfg.get("lora_rank", self.capacity)))
        alpha = float(cfg.get("alpha", cfg.get("lora_alpha", self.default_alpha if rank == self.capacity else rank)))
        if not 1 <= rank <= self.capacity:
            raise ValueError(f"adapter rank {rank} outside 1..{self.capacity} (the server was started with "
                             f"lora_rank {self.capacity})")
        fresh = AdapterState()
        fresh.groups = [{k: v.clone() for k, v in d.items()} for d in self._pristine.groups]
        fresh.meta = dict(self._pristine.meta, rank=rank, alpha=alpha, scaling=alpha / rank)
        if "learning_rate" in cfg:
            fresh.meta["lr"] = float(cfg["learning_rate"])
        if rank < self.capacity:
            self._truncate_rank(fresh, rank)
        self.known.add(model_id)
        try:
            self._put(model_id, fresh)
        except RuntimeError:
            self.known.discard(model_id)
            self.store.pop(model_id, None)
            raise

    def _put(self, model_id: str, st: AdapterState) -> None:
        self.store[model_id] = st
        self.store.move_to_end(model_id)
        while len(self.store) > self.max_adapters - 1:          # one more lives in the engine
            if self.spill_dir:
                victim, vst = next(iter(self.store.items()))     # least recently used; written with its gradients
                os.makedirs(self.spill_dir, exist_ok=True)
                torch.save({"groups": vst.groups, "meta": vst.meta}, self._spill_path(victim))
                del self.store[victim]
                continue
            clean = [k for k, v in self.store.items() if not v.meta.get("epoch_open") and k != model_id]
            if not clean:
                raise RuntimeError("cannot evict an adapter: every resident adapter holds accumulated gradients; "
                                   "call optim_step for one of them first or raise XORL_MAX_ADAPTERS_PER_MODEL")
            del self.store[clean[0]]
            self.known.discard(clean[0])

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

    def session_spec(self, model_id: str) -> Dict[str, Any]:
        meta = self._meta_of(model_id)
        return {"rank": meta.get("rank", self.capacity), "alpha": meta.get("alpha", self.default_alpha),
                "learning_rate": meta.get("lr"), "step": meta.get("step", 0)}

    def _meta_of(self, model_id: str) -> Dict[str, Any]:
        if model_id == self.active:
            r = self.runner
            return {"step": r.step, "lr": float(self.optimizer.lr), "epoch_open": r.epoch_open, **self.session}
        if model_id in self.store:
            return self.store[model_id].meta
        if model_id in self.known and self.spill_dir and os.path.exists(self._spill_path(model_id)):
            return torch.load(self._spill_path(model_id), weights_only=False)["meta"]
        raise KeyError(f"unknown adapter {model_id!r}")

    def set_lr(self, model_id: str, lr: float) -> None:
        if model_id == self.active:
            self.optimizer.set_lr(float(lr))
        elif model_id in self.store:
            self.store[model_id].meta["lr"] = float(lr)
        else:
            raise KeyError(f"adapter {model_id!r} is not resident")

    def get_lr(self, model_id: str) -> float:
        return float(self._meta_of(model_id)["lr"])

    def memory_usage(self) -> Dict[str, int]:
        """Bytes per adapter on this rank: shards of the weights, the gradient and the optimizer state (the
        active adapter's are on the device, the others' in pinned host memory; spilled ones count 0)."""
        active = sum(g.master.numel() * g.master.element_size() + g.grad_shard.numel() * g.grad_shard.element_size()
                     for g in self._groups)
        for per_group in self.optimizer.state.values():
            active += sum(t.numel() * t.element_size() for k, t in per_group.items()
                          if any(k == id(g) for g in self._groups))
        out = {self.active: int(active)}
        for k in self.known:
            if k == self.active:
                continue
            st = self.store.get(k)
            out[k] = int(sum(t.numel() * t.element_size() for d in st.groups for t in d.values())) if st else 0
        return out

    def validate_replica_coherence(self) -> None:
        """With ``XORL_VALIDATE_ADAPTER_REPLICAS=1``: ranks that hold the same shard of the active adapter
        (replica groups of HSDP / DDP) hold the same bits, and every rank agrees on the adapter's counters
        (src/xorl/server/runner/adapters/manager.py:1500-1582)."""
        import torch.distributed as dist
        if os.environ.get("XORL_VALIDATE_ADAPTER_REPLICAS") != "1" or not dist.is_initialized() \
                or dist.get_world_size() <= 1:
            return
        self.engine.sync_optimizer()
        r = self.runner
        dev = self._groups[0].master.device
        counters = torch.tensor([float(r.step), float(self.optimizer.step_count), float(r.epoch_open)],
                                dtype=torch.float64, device=dev)
        lo, hi = counters.clone(), counters.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        if not torch.equal(lo, hi):
            raise RuntimeError(f"adapter {self.active!r}: ranks disagree on its counters ({lo.tolist()} .. {hi.tolist()})")
        for g in self._groups:
            if g.replicate_pg is None:
                continue
            m = g.master.double()
            digest = torch.stack([m.sum(), m.abs().sum(), (m * torch.arange(1, m.numel() + 1, device=dev,
                                                                            dtype=torch.float64)).sum()])
            lo, hi = digest.clone(), digest.clone()
            dist.all_reduce(lo, op=dist.ReduceOp.MIN, group=g.replicate_pg)
            dist.all_reduce(hi, op=dist.ReduceOp.MAX, group=g.replicate_pg)
            if not torch.equal(lo, hi):
                raise RuntimeError(f"adapter {self.active!r}: replicas of {g.name} differ")
