"""Optimizers that update the ZeRO engine's flat fp32 shards in one kernel per shard.

AdamW (fp32 moments), AnyPrecision AdamW (bf16 moments), SGD with
momentum, SignSGD — the optimizer set of src/xorl/optim/optimizer.py:114-242.  The update reads the
clip coefficient from device memory, so a step needs no host synchronisation, and writes the
compute-dtype copy of the weights that the next all-gather sends.
Weight-decay exclusions follow ``no_decay_modules`` (module class names) and ``no_decay_params``
(substring patterns).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch

from ..ops import optim as optim_ops
from ..parallel.zero import FlatParamGroup, Zero3Engine


def _decay_table(engine: Zero3Engine, weight_decay: float, no_decay_modules: Sequence[str],
                 no_decay_params: Sequence[str]) -> Dict[str, float]:
    table: Dict[str, float] = {}
    no_decay_names = set()
    if no_decay_modules:
        for mname, mod in engine.model.named_modules():
            if type(mod).__name__ in no_decay_modules:
                for pname, _ in mod.named_parameters(recurse=False):
                    no_decay_names.add(f"{mname}.{pname}" if mname else pname)
    for g in engine.all_groups():
        for name, _ in g.named_params:
            wd = weight_decay
            if name in no_decay_names or any(pat in name for pat in (no_decay_params or [])):
                wd = 0.0
            table[name] = wd
    return table


class ShardedOptimizer:
    """Base: owns per-group state tensors and iterates (group, segment) pairs."""

    kind = "base"

    def __init__(self, engine: Zero3Engine, lr: float, weight_decay: float = 0.0,
                 no_decay_modules: Sequence[str] = (), no_decay_params: Sequence[str] = ()):
        self.engine = engine
        self.lr = lr
        self.weight_decay = weight_decay
        self.step_count = 0
        self._decay = _decay_table(engine, weight_decay, no_decay_modules, no_decay_params)
        self.state: Dict[str, Dict[int, torch.Tensor]] = {}
        self.lr_scale: Dict[int, float] = {}

    def set_lr(self, lr: float) -> None:
        self.lr = lr

    def _segments(self, g: FlatParamGroup) -> List[Tuple[int, int, float]]:
        """Maximal runs of the shard with equal weight decay (padding inherits its neighbour's)."""
        segs = g.param_segments_in_shard()
        if not segs:
            return [(0, g.shard_numel, 0.0)]
        runs: List[List] = []
        cursor = 0
        for i, a, b in segs:
            wd = self._decay[g.named_params[i][0]]
            if runs and runs[-1][2] == wd:
                runs[-1][1] = b
            else:
                runs.append([cursor, b, wd])
            cursor = b
        runs[-1][1] = g.shard_numel
        # 4-element alignment of run boundaries (vectorised kernel): parameter offsets are multiples
        # of 64 so this only moves boundaries inside alignment padding
        out = []
        for a, b, wd in runs:
            a = (a + 3) // 4 * 4 if a else 0
            out.append((a, b, wd))
        for k in range(len(out) - 1):
            out[k] = (out[k][0], out[k + 1][0], out[k][2])
        return [(a, b, wd) for a, b, wd in out if b > a]

    def _new_state(self, name: str, dtype=torch.float32) -> Dict[int, torch.Tensor]:
        d = {id(g): torch.zeros(g.shard_numel, device=self.engine.device, dtype=dtype)
             for g in self.engine.all_groups() if not getattr(g, "frozen", False)}
        self.state[name] = d
        return d

    def zero_grad(self) -> None:
        self.engine.zero_grad()

    def step(self, clip_coef: Optional[torch.Tensor] = None, grad_scale: float = 1.0) -> None:
        raise NotImplementedError

    # ---- checkpoint ---------------------------------------------------------------------------
    def state_dict(self) -> Dict:
        return {"kind": self.kind, "step": self.step_count, "lr": self.lr}

    def load_state_dict(self, sd: Dict) -> None:
        self.step_count = int(sd.get("step", 0))
        self.lr = float(sd.get("lr", self.lr))


class ShardedAdamW(ShardedOptimizer):
    kind = "adamw"

    def __init__(self, engine, lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0, **kw):
        super().__init__(engine, lr, weight_decay, kw.get("no_decay_modules", ()),
                         kw.get("no_decay_params", ()))
        self.betas, self.eps = betas, eps
        self.exp_avg = self._new_state("exp_avg")
        self.exp_avg_sq = self._new_state("exp_avg_sq")

    def step(self, clip_coef=None, grad_scale: float = 1.0) -> None:
        """One fused kernel per equal-decay run of every shard.  On CUDA the kernels go to the
        engine's optimizer stream, unit by unit in forward order, and the next forward pass waits
        per unit (``Zero3Engine.begin_update``): the bandwidth-bound update overlaps the
        tensor-core-bound start of the next step."""
        from contextlib import nullcontext
        self.step_count += 1
        b1, b2 = self.betas
        eng = self.engine
        side = eng.begin_update((clip_coef,)) if eng.is_cuda else None
        with (torch.cuda.stream(side) if side is not None else nullcontext()):
            for g in eng.all_groups():
                if not g.grad_ready:
                    continue
                m, v = self.exp_avg[id(g)], self.exp_avg_sq[id(g)]
                lp = None if g.shard_lp is g.master else g.shard_lp
                for a, b, wd in self._segments(g):
                    optim_ops.adamw_step_(g.master[a:b], m[a:b], v[a:b], g.grad_shard[a:b],
                                          None if lp is None else lp[a:b], lr=self.lr, beta1=b1, beta2=b2,
                                          eps=self.eps, weight_decay=wd, step=self.step_count,
                                          grad_scale=grad_scale, clip_coef=clip_coef)
                if side is not None:
                    eng.mark_updated(g)


class ShardedAnyPrecisionAdamW(ShardedOptimizer):
    """AdamW with bf16 moments (``optimizer_dtype: bf16``); torch ops on the shard
    (src/xorl/optim/anyprecision_adamw.py).  The reference's Kahan compensation exists for weights
    that are themselves bf16; here the update always lands in the fp32 master shard, so there is no
    rounding of the weight to compensate and no compensation buffer."""
    kind = "anyprecision_adamw"

    def __init__(self, engine, lr, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0,
                 state_dtype=torch.bfloat16, cautious_weight_decay=False, state_cpu_offload: bool = False,
                 denominator_chunk_size: int = 0, **kw):
        """``state_cpu_offload``: the moments live in (pinned) host memory and visit the device one parameter
        group at a time during the step, the next group's moments copied in while the current one updates.
        ``denominator_chunk_size``: elements per pass of the update, which bounds its fp32 temporaries
        (0 = a whole decay segment at once) (src/xorl/optim/anyprecision_adamw.py).  Both leave every bit of
        the result as it is.  The gradient shard is never written by the step: other streams (early norms,
        the next step's gradient kernels) order themselves against reads of it only."""
        super().__init__(engine, lr, weight_decay, kw.get("no_decay_modules", ()),
                         kw.get("no_decay_params", ()))
        self.betas, self.eps, self.cautious = betas, eps, cautious_weight_decay
        self.offload = bool(state_cpu_offload)
        self.chunk = int(denominator_chunk_size or 0)
        self.exp_avg = self._new_state("exp_avg", state_dtype)
        self.exp_avg_sq = self._new_state("exp_avg_sq", state_dtype)
        if self.offload:
            pin = self.engine.device.type == "cuda"
            for d in (self.exp_avg, self.exp_avg_sq):
                for k, t in d.items():
                    d[k] = torch.zeros(t.shape, dtype=t.dtype, device="cpu", pin_memory=pin)
            self._copy_stream = torch.cuda.Stream(self.engine.device) if pin else None

    def _fetch(self, g):
        """Device copies of a group's moments (the tensors themselves when nothing is offloaded)."""
        m, v = self.exp_avg[id(g)], self.exp_avg_sq[id(g)]
        if not self.offload or self.engine.device.type != "cuda":
            return m, v, None
        with torch.cuda.stream(self._copy_stream):
            md, vd = m.to(self.engine.device, non_blocking=True), v.to(self.engine.device, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record()
        return md, vd, ev

    @torch.no_grad()
    def step(self, clip_coef=None, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        b1, b2 = self.betas
        bc1 = 1 - b1 ** self.step_count
        bc2 = 1 - b2 ** self.step_count
        groups = [g for g in self.engine.all_groups() if g.grad_ready and not getattr(g, "frozen", False)]
        nxt = self._fetch(groups[0]) if groups else None
        for gi, g in enumerate(groups):
            m_all, v_all, ready = nxt
            nxt = self._fetch(groups[gi + 1]) if gi + 1 < len(groups) else None      # copied in under this group's update
            if ready is not None:
                cur = torch.cuda.current_stream()
                cur.wait_event(ready)
                m_all.record_stream(cur)          # allocated on the copy stream, used (and freed) under this one
                v_all.record_stream(cur)
            for a0, b0, wd in self._segments(g):
                step_n = self.chunk if self.chunk > 0 else b0 - a0
                for a in range(a0, b0, step_n):
                    b = min(b0, a + step_n)
                    p = g.master[a:b]
                    gr = g.grad_shard[a:b] * grad_scale
                    if clip_coef is not None:
                        gr = gr * clip_coef
                    m = m_all[a:b].float().mul_(b1).add_(gr, alpha=1 - b1)
                    v = v_all[a:b].float().mul_(b2).addcmul_(gr, gr, value=1 - b2)
                    m_all[a:b].copy_(m)
                    v_all[a:b].copy_(v)
                    update = (m / bc1) / ((v / bc2).sqrt_().add_(self.eps))
                    if wd:
                        if self.cautious:
                            mask = (update * p >= 0).to(p.dtype)
                            p.sub_(p * mask, alpha=self.lr * wd)
                        else:
                            p.mul_(1 - self.lr * wd)
                    p.sub_(update, alpha=self.lr)
            if self.offload and m_all is not self.exp_avg[id(g)]:
                self.exp_avg[id(g)].copy_(m_all, non_blocking=True)
                self.exp_avg_sq[id(g)].copy_(v_all, non_blocking=True)
            self.engine.refresh_compute_copy(g)
        if self.offload and self.engine.device.type == "cuda":
            torch.cuda.current_stream().synchronize()         # the host copies are complete before anyone reads them


class ShardedSGD(ShardedOptimizer):
    kind = "sgd"

    def __init__(self, engine, lr, momentum=0.0, nesterov=False, weight_decay=0.0, **kw):
        super().__init__(engine, lr, weight_decay, kw.get("no_decay_modules", ()),
                         kw.get("no_decay_params", ()))
        self.momentum, self.nesterov = momentum, nesterov
        self.buf = self._new_state("momentum_buffer") if momentum else None

    @torch.no_grad()
    def step(self, clip_coef=None, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        for g in self.engine.all_groups():
            if not g.grad_ready:
                continue
            for a, b, wd in self._segments(g):
                p = g.master[a:b]
                gr = g.grad_shard[a:b] * grad_scale
                if clip_coef is not None:
                    gr = gr * clip_coef
                if wd:
                    gr = gr.add(p, alpha=wd)
                if self.buf is not None:
                    mb = self.buf[id(g)][a:b]
                    mb.mul_(self.momentum).add_(gr)
                    gr = gr.add(mb, alpha=self.momentum) if self.nesterov else mb
                p.sub_(gr, alpha=self.lr)
            self.engine.refresh_compute_copy(g)


class ShardedSignSGD(ShardedOptimizer):
    kind = "signsgd"

    def step(self, clip_coef=None, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        for g in self.engine.all_groups():
            if not g.grad_ready:
                continue
            lp = None if g.shard_lp is g.master else g.shard_lp
            for a, b, wd in self._segments(g):
                optim_ops.signsgd_step_(g.master[a:b], g.grad_shard[a:b],
                                        None if lp is None else lp[a:b], lr=self.lr, weight_decay=wd)


class ShardedDistSignSGD(ShardedOptimizer):
    """Majority-vote sign SGD: every data-parallel rank signs the gradient of every micro-batch
    *before* the reduce-scatter, the votes are summed over ranks and micro-batches, and the update is
    ``lr * votes / voters`` -- no second sign (src/xorl/optim/distsignsgd.py: ``DistSignReduceScatter``
    signs the flat buffer, ``DistSignSGD.step`` applies the pre-signed sum).  The engine signs the
    per-micro-batch gradient buffers (``engine.sign_before_reduce``); a shard group of one rank
    accumulates raw gradients in place, so there the single voter signs once at the step."""
    kind = "distsignsgd"

    def __init__(self, engine, lr, weight_decay=0.0, **kw):
        super().__init__(engine, lr, weight_decay, **kw)
        engine.sign_before_reduce = True

    def step(self, clip_coef=None, grad_scale: float = 1.0) -> None:
        self.step_count += 1
        eng = self.engine
        for g in eng.all_groups():
            if not g.grad_ready:
                continue
            if g.world > 1:
                update = g.grad_shard / float(g.world * max(1, eng.micro_batches))
            else:
                update = torch.sign(g.grad_shard)
            for a, b, wd in self._segments(g):
                if wd:
                    g.master[a:b].mul_(1.0 - self.lr * wd)
                g.master[a:b].add_(update[a:b], alpha=-self.lr)
            if g.shard_lp is not g.master:
                g.shard_lp.copy_(g.master)


class MultiOptimizer:
    """Several optimizers driven as one (the reference pairs one optimizer for expert parameters with
    one for the rest, and one per pipeline model part: src/xorl/optim/multi_optimizer.py).  The
    sharded optimizers here already cover every parameter group of an engine; this wrapper exists for
    callers that build optimizers per engine (pipeline stages with virtual chunks) or per parameter
    family and want a single ``step / zero_grad / state_dict`` surface."""

    def __init__(self, optimizers: Dict[str, ShardedOptimizer]):
        if not optimizers:
            raise ValueError("MultiOptimizer needs at least one optimizer")
        self.optimizers = dict(optimizers)

    @property
    def lr(self) -> float:
        return next(iter(self.optimizers.values())).lr

    def set_lr(self, lr: float) -> None:
        for o in self.optimizers.values():
            o.set_lr(lr)

    def zero_grad(self) -> None:
        for o in self.optimizers.values():
            o.zero_grad()

    def step(self, clip_coef=None, grad_scale: float = 1.0) -> None:
        for o in self.optimizers.values():
            o.step(clip_coef=clip_coef, grad_scale=grad_scale)

    def state_dict(self) -> Dict:
        return {name: o.state_dict() for name, o in self.optimizers.items()}

    def load_state_dict(self, sd: Dict) -> None:
        missing = set(self.optimizers) - set(sd)
        if missing:
            raise KeyError(f"optimizer state lacks entries for {sorted(missing)}")
        for name, o in self.optimizers.items():
            o.load_state_dict(sd[name])


def build_optimizer(engine: Zero3Engine, lr: float = 1e-3, betas=(0.9, 0.95), eps: float = 1e-8,
                    weight_decay: float = 1e-2, optimizer_type: str = "adamw",
                    optimizer_dtype: str = "bf16", no_decay_modules=None, no_decay_params=None,
                    optimizer_kwargs: Optional[dict] = None, cautious_weight_decay: bool = False):
    kw = dict(no_decay_modules=no_decay_modules or (), no_decay_params=no_decay_params or ())
    okw = dict(optimizer_kwargs or {})
    any_kw = {k: okw[k] for k in ("state_cpu_offload", "denominator_chunk_size") if okw.get(k)}
    if optimizer_type == "adamw" and not cautious_weight_decay and not any_kw:
        return ShardedAdamW(engine, lr, betas, eps, weight_decay, **kw)
    if optimizer_type in ("adamw", "anyprecision_adamw"):
        dt = torch.float32 if (optimizer_dtype == "fp32" or optimizer_type == "adamw") else torch.bfloat16
        return ShardedAnyPrecisionAdamW(engine, lr, betas, eps, weight_decay, state_dtype=dt,
                                        cautious_weight_decay=cautious_weight_decay, **any_kw, **kw)
    if optimizer_type == "sgd":
        return ShardedSGD(engine, lr, okw.get("momentum", 0.0), okw.get("nesterov", False),
                          weight_decay, **kw)
    if optimizer_type == "signsgd":
        return ShardedSignSGD(engine, lr, weight_decay, **kw)
    if optimizer_type == "distsignsgd":
        return ShardedDistSignSGD(engine, lr, weight_decay, **kw)
    if optimizer_type == "muon":
        from .muon import ShardedMuon
        return ShardedMuon(engine, lr, betas, eps, weight_decay, **okw, **kw)
    raise ValueError(f"unknown optimizer {optimizer_type!r}")
