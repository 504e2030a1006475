"""ZeRO-3 engine on flat per-unit shards.

Replaces the reference's use of ``torch.distributed.fsdp.fully_shard``
(src/xorl/distributed/torch_parallelize.py:333-783) with a runtime that owns the memory layout:

* every *unit* (root = embedding + final norm + lm_head, then one per decoder layer) keeps its
  parameters in one flat buffer; a rank persistently holds only its 1/N slice of the fp32 master
  weights, the two Adam moments, the fp32 gradient accumulator and the compute-dtype copy that is
  all-gathered;
* forward runs unit by unit without an autograd graph and keeps only the unit inputs; backward
  re-gathers a unit, recomputes it under autograd, back-propagates, and immediately reduces that
  unit's gradients into the owners' fp32 accumulators (gradient divide factor 1: losses are
  normalised by the global token count, src/xorl/distributed/torch_parallelize.py:670-672);
* gathers are prefetched one unit ahead on a side stream, gradient reductions overlap the next
  unit's backward.

Transports: ``nccl`` / ``gloo`` collectives (baseline, and the CPU lane) or the fused peer-memory
kernels of ``parallel/symm_transport.py`` when available.
"""
from __future__ import annotations

import os

import math
from contextlib import nullcontext
from typing import Any, Callable, Dict, Iterable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist
from torch import nn

from ..ops import optim as optim_ops
from .state import ParallelState, get_parallel_state

ALIGN = 64  # elements; keeps every parameter and every shard 128-byte aligned in bf16


def _slice_fn(p):
    """This rank's part of the full tensor for a tensor-parallel or expert-parallel parameter."""
    return getattr(p, "_xb_tp_slice", None) or getattr(p, "_xb_ep_slice", None) or getattr(p, "_xb_lmtp_slice", None)


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class FlatParamGroup:
    """Parameters of one unit that share a sharding group (dense vs. expert-parallel)."""

    def __init__(self, name: str, named_params: List[Tuple[str, nn.Parameter]], pg, world: int,
                 rank: int, device: torch.device, compute_dtype: torch.dtype,
                 replicate_pg=None, replicate_world: int = 1):
        self.name = name
        self.named_params = named_params
        self.pg, self.world, self.rank = pg, world, rank
        self.replicate_pg, self.replicate_world = replicate_pg, replicate_world
        self.device, self.compute_dtype = device, compute_dtype
        self.offsets: List[int] = []
        off = 0
        self.shapes = [tuple(getattr(p, "_xb_shape", p.shape)) for _, p in named_params]
        for shp in self.shapes:
            self.offsets.append(off)
            off += _round_up(math.prod(shp), ALIGN)
        self.numel = off
        self.padded = _round_up(max(off, 1), world * ALIGN)
        self.shard_numel = self.padded // world
        # element ranges of the flat layout that belong to no parameter (alignment gaps, tail)
        ends = [o + math.prod(s) for o, s in zip(self.offsets, self.shapes)]
        starts = self.offsets[1:] + [self.padded]
        self.gaps = [(e, n) for e, n in zip(ends, starts) if n > e] if self.offsets else [(0, self.padded)]
        # persistent sharded state
        self.master: torch.Tensor = None      # fp32 [shard]
        self.shard_lp: torch.Tensor = None    # compute dtype [shard] (aliases master when fp32)
        self.grad_shard: torch.Tensor = None  # fp32 [shard]
        self.grad_ready = False               # grad_shard holds this step's accumulated gradient
        # transient
        self.full: Optional[torch.Tensor] = None
        self.full_persistent = False
        self.grad_full: Optional[torch.Tensor] = None
        self.gather_event = None
        self.reduce_event = None
        self.update_event = None              # optimizer kernels of the last step (side stream)
        self.sq: Optional[torch.Tensor] = None  # ||grad shard||^2 of this step, when computed early
        self.sq_valid = False
        self.weight_decay_mask: Optional[List[float]] = None

    # ---- layout helpers ---------------------------------------------------------------------
    def shard_range(self) -> Tuple[int, int]:
        return self.rank * self.shard_numel, (self.rank + 1) * self.shard_numel

    def param_views(self, flat: torch.Tensor) -> List[torch.Tensor]:
        return [flat[o:o + math.prod(s)].view(s) for o, s in zip(self.offsets, self.shapes)]

    def attach_params(self) -> None:
        """Point every parameter at its view of the gathered buffer."""
        for (_, p), v in zip(self.named_params, self.param_views(self.full)):
            p.data = v

    def detach_params(self) -> None:
        empty = torch.empty(0, device=self.device, dtype=self.compute_dtype)
        for _, p in self.named_params:
            p.data = empty

    def zero_grad_gaps(self) -> None:
        """A gathered gradient buffer comes from a pool (or a ring shared with other groups) and
        only the parameter slices are written during backward: what lies between them would be
        summed into the shard by the reduce-scatter and counted in the gradient norm."""
        for a, b in self.gaps:
            self.grad_full[a:b].zero_()

    def attach_grad_views(self, fresh: bool = True) -> None:
        for (_, p), v in zip(self.named_params, self.param_views(self.grad_full)):
            p._xb_grad_buf = v
            p._xb_grad_fresh = fresh
            p.grad = None

    def collect_grads(self) -> None:
        """Zero slices nobody wrote, fold in gradients that arrived through ``p.grad``."""
        for _, p in self.named_params:
            buf = p._xb_grad_buf
            if p.grad is not None:
                if p._xb_grad_fresh:
                    buf.copy_(p.grad)
                else:
                    buf.add_(p.grad.to(buf.dtype))
                p.grad = None
            elif p._xb_grad_fresh:
                buf.zero_()
            p._xb_grad_buf = None
            p._xb_grad_fresh = False

    def param_segments_in_shard(self) -> List[Tuple[int, int, int]]:
        """(param index, start, end) in shard-local coordinates for every overlap."""
        s0, s1 = self.shard_range()
        out = []
        for i, (o, shp) in enumerate(zip(self.offsets, self.shapes)):
            a, b = max(o, s0), min(o + math.prod(shp), s1)
            if a < b:
                out.append((i, a - s0, b - s0))
        return out


class ZeroUnit:
    def __init__(self, name: str, modules: Sequence[nn.Module]):
        self.name = name
        self.modules = list(modules)
        self.groups: List[FlatParamGroup] = []


class _Offloaded:
    """Host copy of a saved activation tuple (pinned), with the events that order the two copies."""
    __slots__ = ("host", "done", "device", "back")

    def __init__(self, host, done):
        self.host, self.done, self.device, self.back = host, done, None, None


class ActivationOffloader:
    """Moves the saved inputs of recomputed layers to pinned host memory on a side stream and brings
    them back one layer ahead of the backward pass (src/xorl/distributed/offloading.py:60-249).
    Pinned buffers are pooled by shape, so after the first step no host allocation happens."""

    def __init__(self, engine):
        self.engine = engine
        self.stream = torch.cuda.Stream() if engine.device.type == "cuda" else None
        self.pool: Dict[Tuple, List[torch.Tensor]] = {}
        self.bytes_offloaded = 0

    def _host_buffer(self, t: torch.Tensor) -> torch.Tensor:
        key = (tuple(t.shape), t.dtype)
        free = self.pool.setdefault(key, [])
        if free:
            return free.pop()
        return torch.empty(t.shape, dtype=t.dtype, device="cpu", pin_memory=self.stream is not None)

    def offload(self, acts):
        if self.stream is None:
            host = tuple(None if a is None else self._host_buffer(a).copy_(a) for a in acts)
            self.bytes_offloaded += sum(h.numel() * h.element_size() for h in host if h is not None)
            return _Offloaded(host, None)
        self.stream.wait_stream(torch.cuda.current_stream())
        host = []
        with torch.cuda.stream(self.stream):
            for a in acts:
                if a is None:
                    host.append(None)
                    continue
                h = self._host_buffer(a)
                h.copy_(a, non_blocking=True)
                a.record_stream(self.stream)
                host.append(h)
                self.bytes_offloaded += h.numel() * h.element_size()
            done = torch.cuda.Event()
            done.record(self.stream)
        return _Offloaded(tuple(host), done)

    def prefetch(self, item) -> None:
        if not isinstance(item, _Offloaded) or item.device is not None:
            return
        dev = self.engine.device
        if self.stream is None:
            item.device = tuple(None if h is None else h.to(dev) for h in item.host)
            return
        with torch.cuda.stream(self.stream):
            self.stream.wait_event(item.done)
            item.device = tuple(None if h is None else h.to(dev, non_blocking=True) for h in item.host)
            item.back = torch.cuda.Event()
            item.back.record(self.stream)

    def fetch(self, item):
        if not isinstance(item, _Offloaded):
            return item
        self.prefetch(item)
        if item.back is not None:
            torch.cuda.current_stream().wait_event(item.back)
            for d in item.device:
                if d is not None:
                    d.record_stream(torch.cuda.current_stream())
        for h in item.host:
            if h is not None:
                self.pool.setdefault((tuple(h.shape), h.dtype), []).append(h)
        return item.device


class Zero3Engine:
    """Runs forward/backward unit by unit with ZeRO-3 sharding (world >= 1)."""

    def __init__(self, model: nn.Module, pstate: Optional[ParallelState] = None, *,
                 compute_dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None,
                 reduce_dtype: torch.dtype = torch.float32, reshard_after_forward: bool = True,
                 activation_offload: bool = False,
                 recompute: bool = True, seed: int = 0, comm_backend: str = "nccl",
                 shard: bool = True, forward_prefetch: bool = True, backward_prefetch: bool = True,
                 moe_grad_reduce_mode: Optional[str] = None):
        self.model = model
        self.ps = pstate or get_parallel_state()
        self.device = device or torch.device("cuda" if torch.cuda.is_available() else "cpu")
        self.compute_dtype = compute_dtype
        self.reduce_dtype = reduce_dtype
        # train.moe_grad_reduce_mode: "bf16_a2a_fp32_sum" sends expert gradients as stochastically rounded
        # bf16 through an all-to-all and sums the received slices in fp32; "reduce_scatter" is the
        # plain collective in the reduce dtype (src/xorl/distributed/fsdp2/bf16_a2a_reduce.py:64-114)
        self.moe_grad_reduce_mode = moe_grad_reduce_mode
        self.bf16_a2a_reduce = os.environ.get("XORL_B200_BF16_A2A_REDUCE", "1") == "1"
        self.forward_prefetch, self.backward_prefetch = forward_prefetch, backward_prefetch
        self.offloader = ActivationOffloader(self) if activation_offload else None
        self.expert_load_tracker = None      # utils.moe_metrics.ExpertLoadTracker, attached by the trainer / runner
        self.recompute = recompute
        self.comm_backend = comm_backend
        self.is_cuda = self.device.type == "cuda"
        ps = self.ps
        if shard and ps.dp_mode == "fsdp2":
            self.shard_pg, self.shard_world = ps.group("fsdp"), ps.size("fsdp") if "fsdp" in ps.groups else 1
            self.shard_rank = ps.rank_in("fsdp")
            self.rep_pg = ps.group("dp_replicate")
            self.rep_world = ps.dp_replicate_size
            self.sp_sync_pg = ps.group("sp_grad_sync")
        else:
            # ddp / none: every rank holds everything, gradients are all-reduced over dp x sp
            self.shard_pg, self.shard_world, self.shard_rank = None, 1, 0
            self.rep_pg, self.rep_world = ps.group("dp_sp"), ps.size("dp_sp") if "dp_sp" in ps.groups else 1
            self.sp_sync_pg = None
        self.ep_shard_pg = ps.group("ep_fsdp")
        self.ep_shard_world = ps.ep_fsdp_size if ps.ep_size > 1 else self.shard_world
        self.ep_shard_rank = ps.rank_in("ep_fsdp") if ps.ep_size > 1 else self.shard_rank
        self.reshard = reshard_after_forward and self.shard_world > 1
        self.sign_before_reduce = False        # set by the majority-vote sign SGD optimizer
        self.micro_batches = 0                 # forward_backward calls since zero_grad
        self.units: List[ZeroUnit] = []
        self.comm_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        # The optimizer's kernels are bandwidth-bound and the next forward pass is tensor-core
        # bound: they run side by side.  The update of step t is issued on ``opt_stream`` unit by
        # unit in forward order, and step t+1 waits per unit (before it reads the unit's parameters
        # or overwrites its gradient shard), not for the whole update.
        self.overlap_optimizer = self.is_cuda and os.environ.get("XORL_B200_OVERLAP_OPTIMIZER", "1") == "1"
        self.opt_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self._opt_pending = False
        # Squared gradient norms are taken per unit as soon as the unit's gradient is final (last
        # micro-batch only), on a side stream, instead of in one pass after backward.
        self.early_grad_norm = os.environ.get("XORL_B200_EARLY_GRAD_NORM", "1") == "1"
        self.final_micro_batch = True          # callers with gradient accumulation set this per micro-batch
        self.norm_stream = torch.cuda.Stream(device=self.device) if self.is_cuda else None
        self._full_pool: Dict[Tuple[int, torch.dtype], List[torch.Tensor]] = {}
        self._build_units(seed)
        self.symm = None  # fused peer-memory transport (attach_peer_transport)

    # ---------------------------------------------------------------------------------------
    # construction
    # ---------------------------------------------------------------------------------------
    def _swap_parameters(self) -> None:
        """Replaces every parameter (meta or real) by a storage-less parameter on the engine's
        device; the original shape and, for real tensors, the initial values are kept on the new
        object until the unit is materialised.  Tied parameters stay tied."""
        mapping: Dict[int, nn.Parameter] = {}
        for mod in self.model.modules():
            for k, p in list(mod._parameters.items()):
                if p is None:
                    continue
                if id(p) not in mapping:
                    newp = nn.Parameter(torch.empty(0, device=self.device, dtype=self.compute_dtype),
                                        requires_grad=p.requires_grad)
                    newp._xb_shape = tuple(p.shape)
                    newp._xb_init = None if p.is_meta else p.detach()
                    for attr in ("_xb_expert", "_xb_tp", "_xb_no_decay", "_xb_full_shape",
                                 "_xb_tp_slice", "_xb_tp_reduce", "_xb_materialize", "_xb_lora", "_xb_ep",
                                 "_xb_ep_slice", "_xb_lmtp", "_xb_lmtp_slice"):
                        if hasattr(p, attr):
                            setattr(newp, attr, getattr(p, attr))
                    mapping[id(p)] = newp
                mod._parameters[k] = mapping[id(p)]

    def _build_units(self, seed: int) -> None:
        model = self.model
        self._swap_parameters()
        seen: set = set()
        fqn_of = {id(p): n for n, p in model.named_parameters()}
        index_of = {n: i for i, (n, _) in enumerate(model.named_parameters())}
        cfg = getattr(model, "config", None)
        std = getattr(cfg, "initializer_range", 0.02)
        zc = getattr(cfg, "zero_centered_norm", False)
        from ..models.decoder import init_parameter_ as _init_plain
        lora_cfg = getattr(model, "_xb_lora_config", None) or {}
        b_std, b_seed = float(lora_cfg.get("b_init_std") or 0.0), int(lora_cfg.get("b_init_seed") or 0)

        def init_parameter_(name, p, *a, **k):
            # lora.lora_b_init_std: B starts as N(0, std) instead of zero (drawn from lora_b_init_seed)
            if b_std > 0 and (".lora_B." in name or name.endswith("_lora_B")) and not p.is_meta:
                from ..adapters.lora import init_lora_parameter_
                return init_lora_parameter_(name, p, 0, b_seed, b_std)
            return _init_plain(name, p, *a, **k)

        for uname, mods in model.unit_modules():
            unit = ZeroUnit(uname, mods)
            dense: List[Tuple[str, nn.Parameter]] = []
            expert: List[Tuple[str, nn.Parameter]] = []
            frozen: List[Tuple[str, nn.Parameter]] = []
            frozen_expert: List[Tuple[str, nn.Parameter]] = []   # frozen expert weights (adapters over experts)
            head: List[Tuple[str, nn.Parameter]] = []       # lm-head rows under lm-head-only tensor parallelism
            for m in mods:
                for p in m.parameters():
                    if id(p) in seen or not p.requires_grad and False:
                        continue
                    seen.add(id(p))
                    if getattr(p, "_xb_lmtp", None) is not None:
                        head.append((fqn_of[id(p)], p))
                    elif not p.requires_grad:
                        # expert-parallel slices differ from rank to rank of the data-parallel group: frozen or
                        # not, they are sharded over the ranks that hold the same experts
                        (frozen_expert if getattr(p, "_xb_expert", False) and self.ps.ep_size > 1
                         else frozen).append((fqn_of[id(p)], p))
                    else:
                        (expert if getattr(p, "_xb_expert", False) else dense).append((fqn_of[id(p)], p))
            for kind, plist in (("dense", dense), ("expert", expert), ("frozen", frozen),
                                ("frozen_expert", frozen_expert), ("head", head)):
                if not plist:
                    continue
                if kind == "head":
                    # sharded over the ranks that hold the same vocabulary rows
                    hp = self.ps.group("lm_head_replica") if self.shard_pg is not None else None
                    g = FlatParamGroup(f"{uname}.{kind}", plist, hp, self.ps.size("lm_head_replica") if hp is not None else 1,
                                       self.ps.rank_in("lm_head_replica") if hp is not None else 0, self.device,
                                       self.compute_dtype,
                                       None if hp is not None else self.ps.group("lm_head_replica"),
                                       1 if hp is not None else self.ps.size("lm_head_replica"))
                elif kind in ("expert", "frozen_expert") and self.ps.ep_size > 1:
                    g = FlatParamGroup(f"{uname}.{kind}", plist, self.ep_shard_pg, self.ep_shard_world,
                                       self.ep_shard_rank, self.device, self.compute_dtype)
                else:
                    g = FlatParamGroup(f"{uname}.{kind}", plist, self.shard_pg, self.shard_world,
                                       self.shard_rank, self.device, self.compute_dtype,
                                       self.rep_pg, self.rep_world)
                g.is_expert = kind in ("expert", "frozen_expert")
                g.is_head = kind == "head"
                g.frozen = kind in ("frozen", "frozen_expert") or (kind == "head" and not plist[0][1].requires_grad)
                self._materialize_group(g, std, seed, index_of, zc, init_parameter_)
                unit.groups.append(g)
            self.units.append(unit)
        leftover = [n for n, p in model.named_parameters() if id(p) not in seen]
        if leftover:
            raise RuntimeError(f"parameters not covered by any ZeRO unit: {leftover[:5]}")
        # move buffers (rotary tables etc.)
        for m in model.modules():
            for k, b in list(m._buffers.items()):
                if b is not None and b.device != self.device and not b.is_meta:
                    m._buffers[k] = b.to(self.device)

    def attach_peer_transport(self, required: bool = False) -> bool:
        """Moves the compute-dtype shards into a symmetric heap and switches parameter gathers and gradient
        reduce-scatters to the framework's own kernels / copy-engine transfers over peer memory
        (``parallel/symm_transport.py``).  Returns False (and keeps the collective library) when peer
        mapping is not available, unless ``required``."""
        try:
            from .symm_transport import SymmetricTransport
            self.symm = SymmetricTransport.create(self)
            return self.symm is not None
        except Exception as e:  # noqa: BLE001
            if required:
                raise
            from ..utils.logging import warning_rank0
            warning_rank0(f"fused peer-memory transport unavailable ({e!r}); using NCCL collectives")
            self.symm = None
            return False

    def _materialize_group(self, g: FlatParamGroup, std, seed, index_of, zc, init_fn) -> None:
        """Builds the unit's full fp32 image once (initialising meta parameters in place), keeps
        this rank's slice as master weights and drops the rest."""
        if getattr(g, "frozen", False):
            self._materialize_frozen(g, std, seed, index_of, zc, init_fn)
            return
        full32 = torch.zeros(g.padded, device=self.device, dtype=torch.float32)
        for (name, p), view in zip(g.named_params, g.param_views(full32)):
            init = getattr(p, "_xb_init", None)
            tp_slice = _slice_fn(p)
            if init is None and tp_slice is not None:
                # tensor- or expert-parallel shard: draw the full tensor, keep this rank's slice
                full = torch.empty(p._xb_full_shape, device=self.device, dtype=torch.float32)
                init_fn(name, full, std, seed, index_of[name], zc)
                view.copy_(tp_slice(full))
                del full
            elif init is None:
                init_fn(name, view, std, seed, index_of[name], zc)
            else:
                view.copy_(init.to(device=self.device, dtype=torch.float32))
                p._xb_init = None
        s0, s1 = g.shard_range()
        g.master = full32[s0:s1].clone()
        g.shard_lp = g.master if self.compute_dtype == torch.float32 else g.master.to(self.compute_dtype)
        g.grad_shard = torch.zeros(g.shard_numel, device=self.device, dtype=torch.float32)
        del full32
        if g.world == 1:
            g.full = g.shard_lp
            g.full_persistent = True
            g.attach_params()

    def _materialize_frozen(self, g: FlatParamGroup, std, seed, index_of, zc, init_fn) -> None:
        """Frozen parameters (LoRA / QLoRA bases) keep only the compute-dtype shard: no master copy,
        no gradient accumulator, no optimizer state.  A parameter may bring its own
        ``_xb_materialize(shape, device)`` producing the exact bits to store (packed quantised data
        reinterpreted in the compute dtype)."""
        full = torch.zeros(g.padded, device=self.device, dtype=self.compute_dtype)
        for (name, p), view in zip(g.named_params, g.param_views(full)):
            mat = getattr(p, "_xb_materialize", None)
            init = getattr(p, "_xb_init", None)
            if mat is not None:
                view.copy_(mat(view.shape, self.device, name, seed))
            elif init is not None:
                view.copy_(init.to(device=self.device, dtype=self.compute_dtype))
                p._xb_init = None
            else:
                tmp = torch.empty(view.shape, device=self.device, dtype=torch.float32)
                tp_slice = _slice_fn(p)
                if tp_slice is not None:
                    fullp = torch.empty(p._xb_full_shape, device=self.device, dtype=torch.float32)
                    init_fn(name, fullp, std, seed, index_of[name], zc)
                    tmp.copy_(tp_slice(fullp))
                else:
                    init_fn(name, tmp, std, seed, index_of[name], zc)
                view.copy_(tmp)
        s0, s1 = g.shard_range()
        g.master = None
        g.shard_lp = full[s0:s1].clone()
        g.grad_shard = None
        if g.world == 1:
            g.full = g.shard_lp
            g.full_persistent = True
            g.attach_params()

    # ---------------------------------------------------------------------------------------
    # optimizer overlap
    # ---------------------------------------------------------------------------------------
    def begin_update(self, tensors=()):
        """Stream on which an optimizer should issue its kernels (None: the current stream).  The
        side stream first waits for everything issued so far (gradients, clip coefficient)."""
        if not (self.overlap_optimizer and self.symm is None):
            return None
        cur = torch.cuda.current_stream()
        self.opt_stream.wait_stream(cur)
        for t in tensors:
            if t is not None and t.is_cuda:
                t.record_stream(self.opt_stream)
        self._opt_pending = True
        return self.opt_stream

    def mark_updated(self, g: FlatParamGroup) -> None:
        """Called on the optimizer's stream after the last kernel that touches group ``g``."""
        if self._opt_pending:
            g.update_event = torch.cuda.Event()
            g.update_event.record(self.opt_stream)

    def _wait_update(self, g: FlatParamGroup, stream=None) -> None:
        ev = g.update_event
        if ev is not None:
            (stream or torch.cuda.current_stream()).wait_event(ev)

    def sync_optimizer(self) -> None:
        """Makes the current stream wait for every pending optimizer kernel (anything that reads or
        writes shards outside the forward / backward path calls this first)."""
        if self._opt_pending:
            torch.cuda.current_stream().wait_stream(self.opt_stream)
            for g in self.all_groups():
                g.update_event = None
            self._opt_pending = False

    # ---------------------------------------------------------------------------------------
    # gather / release
    # ---------------------------------------------------------------------------------------
    def _take_full(self, numel: int, dtype: torch.dtype, on_comm_stream: bool = False) -> torch.Tensor:
        """Buffers cycle between parameter gathers (written on the side stream) and gradient
        buffers (written on the compute stream).  An entry remembers the side-stream event of its
        last use there; a compute-side taker waits for it."""
        pool = self._full_pool.setdefault((numel, dtype), [])
        if pool:
            t, ev = pool.pop()
            if ev is not None and not on_comm_stream:
                torch.cuda.current_stream().wait_event(ev)
            return t
        return torch.empty(numel, device=self.device, dtype=dtype)

    def _give_full(self, t: torch.Tensor, comm_event=None) -> None:
        self._full_pool.setdefault((t.numel(), t.dtype), []).append((t, comm_event))

    def gather(self, unit: ZeroUnit, async_op: bool = True) -> None:
        """Start (or no-op if already resident) the all-gather of a unit's parameters."""
        for g in unit.groups:
            if g.full is not None:
                continue
            g.full = self._take_full(g.padded, self.compute_dtype, on_comm_stream=True)
            if self.is_cuda:
                self._wait_update(g, self.comm_stream)
            if self.symm is not None and self.symm.can_gather(g):
                self.symm.all_gather(g, self.comm_stream)
            elif self.is_cuda:
                self.comm_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.comm_stream):
                    dist.all_gather_into_tensor(g.full, g.shard_lp, group=g.pg)
                    g.gather_event = torch.cuda.Event()
                    g.gather_event.record(self.comm_stream)
            else:
                dist.all_gather_into_tensor(g.full, g.shard_lp, group=g.pg)

    def wait_gather(self, unit: ZeroUnit) -> None:
        for g in unit.groups:
            if g.full_persistent:
                self._wait_update(g)          # single owner: the optimizer wrote these weights in place
            if g.gather_event is not None:
                torch.cuda.current_stream().wait_event(g.gather_event)
                g.gather_event = None
            g.attach_params()

    def release(self, unit: ZeroUnit) -> None:
        for g in unit.groups:
            if g.full_persistent or g.full is None:
                continue
            g.detach_params()
            if self.is_cuda:
                # the buffer may be re-filled by the side stream only after compute is done with it
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
                self.comm_stream.wait_event(ev)
            self._give_full(g.full)
            g.full = None

    # ---------------------------------------------------------------------------------------
    # gradient reduction
    # ---------------------------------------------------------------------------------------
    def _prepare_grad_buffers(self, unit: ZeroUnit) -> None:
        for g in unit.groups:
            if getattr(g, "frozen", False):
                continue
            self._wait_update(g)              # the last optimizer step still reads this gradient shard
            g.sq_valid = False
            if g.world == 1:
                # single owner: kernels write (or accumulate) straight into the fp32 accumulator
                g.grad_full = g.grad_shard
                g.attach_grad_views(fresh=not g.grad_ready)
            elif self.symm is not None and self.symm.can_reduce(g):
                g.grad_full = self.symm.take_grad_buffer(g)
                g.zero_grad_gaps()
                g.attach_grad_views()
            else:
                g.grad_full = self._take_full(g.padded, self.compute_dtype)
                g.zero_grad_gaps()
                g.attach_grad_views()

    def _reduce_unit_grads(self, unit: ZeroUnit, collected: bool = False) -> None:
        for g in unit.groups:
            if getattr(g, "frozen", False):
                continue
            if not collected:
                g.collect_grads()
            accumulate = g.grad_ready
            gf = g.grad_full
            if self.sign_before_reduce and g.world > 1:
                # majority-vote sign SGD: each rank votes with the sign of its micro-batch gradient
                # (exact sums over sequence-parallel ranks come first)
                if self.sp_sync_pg is not None and not getattr(g, "is_expert", False):
                    dist.all_reduce(gf, group=self.sp_sync_pg)
                gf.sign_()
            if self.ps.tp_size > 1 and self.ps.group("tp") is not None and g.world > 1:
                # (with a shard group of one the gradients accumulate in place over micro-batches:
                # their sum over the tensor-parallel group is taken once, in finish_grad_sync)
                for (_, p), v in zip(g.named_params, g.param_views(gf)):
                    if getattr(p, "_xb_tp_reduce", False):
                        dist.all_reduce(v, group=self.ps.group("tp"))
            early = self._early_norm_ok(g)
            if g.world == 1:
                # gradients were produced in place in g.grad_shard
                if early:
                    ev = torch.cuda.Event()
                    ev.record(torch.cuda.current_stream())
                    self.norm_stream.wait_event(ev)
                    with torch.cuda.stream(self.norm_stream):
                        self._group_sumsq(g)
            elif self.symm is not None and self.symm.can_reduce(g):
                g.sq_valid = False
                self.symm.reduce_scatter_accumulate(g, gf, accumulate, self.comm_stream)
                if early and not g.sq_valid:
                    with torch.cuda.stream(self.comm_stream):
                        self._group_sumsq(g)
            elif self.is_cuda:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
                self.comm_stream.wait_event(ev)
                with torch.cuda.stream(self.comm_stream):
                    self._rs_collective(g, gf, accumulate)
                    if early:
                        self._group_sumsq(g)
                    g.reduce_event = torch.cuda.Event()
                    g.reduce_event.record(self.comm_stream)
                self._give_full(gf, g.reduce_event)
            else:
                self._rs_collective(g, gf, accumulate)
                self._give_full(gf)
            g.grad_full = None
            g.grad_ready = True

    def _early_norm_ok(self, g: FlatParamGroup) -> bool:
        """The shard's squared norm may be taken right after this reduction: it is the step's last
        micro-batch and nothing later in the step (replica / sequence-parallel / tensor-parallel
        all-reduces of finish_grad_sync, sign votes) changes the shard again."""
        if not (self.is_cuda and self.early_grad_norm and self.final_micro_batch):
            return False
        if self.sign_before_reduce or self.ps.tp_size > 1:
            return False
        if g.replicate_pg is not None and g.replicate_world > 1:
            return False
        if self.sp_sync_pg is not None and not getattr(g, "is_expert", False):
            return False
        return True

    def _group_sumsq(self, g: FlatParamGroup) -> None:
        if g.sq is None:
            g.sq = torch.zeros(1, device=self.device, dtype=torch.float32)
        optim_ops.sumsq_(g.grad_shard, g.sq, False)
        g.sq_valid = True

    def _rs_collective(self, g: FlatParamGroup, gf: torch.Tensor, accumulate: bool) -> None:
        a2a = self.reduce_dtype == torch.bfloat16 and self.bf16_a2a_reduce
        if getattr(g, "is_expert", False) and self.moe_grad_reduce_mode is not None:
            a2a = self.moe_grad_reduce_mode == "bf16_a2a_fp32_sum"
        if a2a and gf.dtype == torch.float32:
            # bf16 on the wire, stochastic rounding on the way out, fp32 summation on arrival
            from .dist_utils import stochastic_bf16_all_to_all_reduce_scatter
            stochastic_bf16_all_to_all_reduce_scatter(gf, g.grad_shard, g.pg, accumulate)
            return
        src = gf if gf.dtype == self.reduce_dtype else gf.to(self.reduce_dtype)
        out = torch.empty(g.shard_numel, device=self.device, dtype=src.dtype)
        dist.reduce_scatter_tensor(out, src, op=dist.ReduceOp.SUM, group=g.pg)
        if accumulate:
            g.grad_shard.add_(out)
        else:
            g.grad_shard.copy_(out)

    def finish_grad_sync(self) -> None:
        """Wait for outstanding reductions; all-reduce over replicas (HSDP / DDP) and over
        sequence-parallel ranks that are not part of the shard group."""
        if self.is_cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        for unit in self.units:
            for g in unit.groups:
                g.reduce_event = None
                if g.grad_shard is None:
                    continue
                if g.world == 1 and self.ps.tp_size > 1 and self.ps.group("tp") is not None:
                    for i, a, b in g.param_segments_in_shard():
                        if getattr(g.named_params[i][1], "_xb_tp_reduce", False):
                            dist.all_reduce(g.grad_shard[a:b], group=self.ps.group("tp"))
                if g.replicate_pg is not None and g.replicate_world > 1:
                    dist.all_reduce(g.grad_shard, group=g.replicate_pg)
                if self.sp_sync_pg is not None and not getattr(g, "is_expert", False) and not \
                        (self.sign_before_reduce and g.world > 1):
                    dist.all_reduce(g.grad_shard, group=self.sp_sync_pg)

    def zero_grad(self) -> None:
        # called once per optimizer step, before the first forward that sees the new weights:
        # quantised copies of the weights (block fp8 experts) made from the old ones are stale
        from ..ops.fp8_grouped import invalidate_weight_cache
        invalidate_weight_cache()
        self.micro_batches = 0
        if self.symm is not None:
            self.sync_optimizer()
            # parameter shards were rewritten by the optimizer: no peer may read them earlier
            self.symm.step_barrier(torch.cuda.current_stream())
        for unit in self.units:
            for g in unit.groups:
                g.grad_ready = False

    # ---------------------------------------------------------------------------------------
    # forward / backward over one micro-batch
    # ---------------------------------------------------------------------------------------
    def _units_by_role(self):
        root = next((u for u in self.units if u.name == "root"), None)
        layers = [u for u in self.units if u.name != "root"]
        return root, layers

    # ---- primitives shared by the plain step and the pipeline runner ----------------------------
    def make_step_context(self, input_ids, position_ids=None, cu_seqlens=None, grad_scale: float = 1.0,
                          extra=None):
        model = self.model
        ctx = model.make_context(input_ids, position_ids, cu_seqlens, training=True, extra=extra)
        if getattr(model, "aux_loss_enabled", False):
            # per-layer auxiliary losses are weighted like a token mean over the global batch
            ctx.aux["aux_loss_scale"] = float(ctx.num_tokens) * grad_scale
        # record expert choices in the first pass and replay them when a layer is recomputed, so
        # both passes dispatch identically (src/xorl/models/layers/moe/routing_replay.py)
        ctx.aux["record_routing"] = self.recompute
        # the fused EP path reuses its peer-memory workspaces across layers, which is only safe when
        # a layer's backward immediately follows its (re)computed forward
        ctx.aux["ep_workspace_reuse_ok"] = self.recompute
        if getattr(self, "expert_load_tracker", None) is not None and self.expert_load_tracker.enabled:
            ctx.aux["collect_expert_load"] = True
        return ctx

    def _take_expert_load(self, ctx, lidx: int) -> None:
        """Moves a layer's per-expert token counts (first forward pass only) to the tracker."""
        load = ctx.aux.pop(("expert_load", lidx), None)
        tracker = getattr(self, "expert_load_tracker", None)
        if load is not None and tracker is not None:
            tracker.add(lidx, load)

    def chunk_forward(self, layers: List[ZeroUnit], acts, ctx, keep_last_gathered: bool = False):
        """Forward through consecutive layer units.  Returns (acts_out, saved) where ``saved`` is
        what ``chunk_backward`` needs (unit inputs when recomputing, autograd graphs otherwise)."""
        nl = len(layers)
        saved: List = []
        if nl:
            self.gather(layers[0])
        for i, unit in enumerate(layers):
            self.gather(unit)
            self.wait_gather(unit)
            if i + 1 < nl and self.forward_prefetch:
                self.gather(layers[i + 1])
            layer = unit.modules[0]
            if self.recompute:
                saved.append(self.offloader.offload(acts) if self.offloader is not None else acts)
                with torch.no_grad():
                    acts = layer(*acts, ctx)
            else:
                ins = tuple(a.detach().requires_grad_() if a is not None else None for a in acts)
                with torch.enable_grad():
                    outs = layer(*ins, ctx)
                saved.append((ins, outs))
                acts = tuple(o.detach() if o is not None else None for o in outs)
            if ctx.aux.get("collect_expert_load"):
                self._take_expert_load(ctx, getattr(layer, "layer_idx", i))
            if self.reshard and self.recompute and not (keep_last_gathered and i == nl - 1):
                self.release(unit)
        return acts, saved

    def chunk_backward(self, layers: List[ZeroUnit], saved: List, dacts, ctx, defer_reduce: bool = False):
        """Backward through the same units, last to first.  Returns (dacts_in, pending) where
        ``pending`` lists the units whose gradient reduction was deferred (``defer_reduce``)."""
        nl = len(layers)
        pending: List = []
        for i in range(nl - 1, -1, -1):
            unit = layers[i]
            self.gather(unit)
            self.wait_gather(unit)
            if i > 0 and self.backward_prefetch:
                self.gather(layers[i - 1])
            self._prepare_grad_buffers(unit)
            layer = unit.modules[0]
            lidx = getattr(layer, "layer_idx", i)
            if self.recompute:
                if self.offloader is not None:
                    if i > 0:
                        self.offloader.prefetch(saved[i - 1])
                    saved[i] = self.offloader.fetch(saved[i])
                ins = tuple(a.detach().requires_grad_() if a is not None else None for a in saved[i])
                saved[i] = None
                ctx.aux["record_routing"] = False
                ctx.aux["collect_expert_load"] = False          # counted in the first pass already
                rec = ctx.aux.pop(("routing_record", lidx), None)
                if rec is not None:
                    ctx.aux[("routing_replay", lidx)] = rec
                with torch.enable_grad():
                    outs = layer(*ins, ctx)
            else:
                ins, outs = saved[i]
                saved[i] = None
            pairs = [(o, d) for o, d in zip(outs, dacts) if o is not None and d is not None]
            aux = ctx.aux.pop(("aux_loss", lidx), None)
            ctx.aux.pop(("routing_replay", lidx), None)
            tensors = [o for o, _ in pairs]
            grads = [d for _, d in pairs]
            if aux is not None:
                tensors.append(aux)
                grads.append(torch.ones_like(aux))
            torch.autograd.backward(tensors, grads)
            if self.is_cuda:
                from ..ops.grad_sink import join_wgrad_stream
                join_wgrad_stream()          # weight-gradient GEMMs issued on their side stream
            dacts = tuple(a.grad if a is not None else None for a in ins)
            del ins, outs, pairs, tensors, grads
            if defer_reduce:
                pending.append(self._detach_grad_buffers(unit))
            else:
                self._reduce_unit_grads(unit)
            if self.reshard:
                self.release(unit)
        return dacts, pending

    def _detach_grad_buffers(self, unit: ZeroUnit):
        """Fold straggler gradients now, but keep the unit's gradient buffers alive for weight
        gradients that will be produced later (zero-bubble schedules)."""
        rec = []
        for g in unit.groups:
            if getattr(g, "frozen", False):
                continue
            g.collect_grads()
            rec.append((g, g.grad_full))
            g.grad_full = None
            if g.world == 1:
                # gradients are produced in place in the accumulator: later micro-batches must add
                g.grad_ready = True
        return unit, rec

    def reduce_deferred(self, pending: List) -> None:
        for unit, rec in pending:
            for g, gf in rec:
                g.grad_full = gf
                # collect_grads already ran; _reduce_unit_grads calls it again on cleared attrs
                for _, p in g.named_params:
                    p._xb_grad_buf = None
                    p._xb_grad_fresh = False
            self._reduce_unit_grads(unit, collected=True)

    def head_forward_backward(self, acts, labels, ctx, grad_scale, extra_loss_fn=None):
        """Final norm + lm-head loss, forward and backward at once.  Returns (loss, dacts)."""
        head_in = tuple(a.detach().requires_grad_() if a is not None else None for a in acts)
        with torch.enable_grad():
            loss = self.model.head_loss(*head_in, labels, ctx, grad_scale)
            total = loss
            if extra_loss_fn is not None:
                extra = extra_loss_fn(ctx)
                if extra is not None:
                    total = total + extra
            total.backward()
        if self.is_cuda:
            from ..ops.grad_sink import join_wgrad_stream
            join_wgrad_stream()
        return loss.detach(), tuple(a.grad if a is not None else None for a in head_in)

    def embed_backward(self, input_ids, ctx, dacts) -> None:
        with torch.enable_grad():
            emb = self.model.forward_embed(input_ids, ctx)
        pairs = [(o, d) for o, d in zip(emb, dacts) if o is not None and d is not None]
        if pairs and pairs[0][0].requires_grad:
            torch.autograd.backward([o for o, _ in pairs], [d for _, d in pairs])
        if self.is_cuda:
            from ..ops.grad_sink import join_wgrad_stream
            join_wgrad_stream()

    def forward_backward(self, input_ids: torch.Tensor, labels: torch.Tensor, *,
                         position_ids=None, cu_seqlens=None, grad_scale: float = 1.0,
                         extra_loss_fn: Optional[Callable] = None, extra=None) -> torch.Tensor:
        """One micro-batch.  Returns ``grad_scale * sum(token CE)`` (detached).  Gradients are
        accumulated into the fp32 shards; call ``finish_grad_sync`` after the last micro-batch."""
        model = self.model
        self.micro_batches += 1
        root, layers = self._units_by_role()
        self.gather(root)
        self.wait_gather(root)
        ctx = self.make_step_context(input_ids, position_ids, cu_seqlens, grad_scale, extra)
        with torch.no_grad():
            acts = model.forward_embed(input_ids, ctx)
        acts, saved = self.chunk_forward(layers, acts, ctx, keep_last_gathered=True)
        self._prepare_grad_buffers(root)
        loss_value, dacts = self.head_forward_backward(acts, labels, ctx, grad_scale, extra_loss_fn)
        dacts, _ = self.chunk_backward(layers, saved, dacts, ctx)
        self.embed_backward(input_ids, ctx, dacts)
        self._reduce_unit_grads(root)
        if self.reshard:
            self.release(root)
        return loss_value

    @torch.no_grad()
    @torch.no_grad()
    def eval_loss(self, input_ids, labels, *, position_ids=None, cu_seqlens=None) -> Tuple[torch.Tensor, torch.Tensor]:
        """(sum of the next-token negative log-likelihoods over supervised labels, their count) of this
        rank's batch, without gradients.  Built for data-parallel layouts (every rank holds whole
        sequences and the whole vocabulary)."""
        if self.ps.tp_size > 1 or self.ps.pp_size > 1 or self.ps.ulysses_size * self.ps.ringattn_size > 1 \
                or getattr(self.ps, "lm_head_tp_size", 1) > 1:
            raise NotImplementedError("evaluation runs on data-parallel layouts (no tensor, pipeline, context or "
                                      "lm-head parallelism)")
        from ..ops.loss import fused_linear_token_loss
        hidden = self.forward_only(input_ids, position_ids=position_ids, cu_seqlens=cu_seqlens)
        root, _ = self._units_by_role()
        self.gather(root)
        self.wait_gather(root)
        head = self.model.lm_head.weight if hasattr(self.model, "lm_head") else self.model.embed_tokens.weight
        _, lp, _ = fused_linear_token_loss(hidden, head, labels, lambda lp, mask: (lp.sum() * 0, {}), 1.0)
        valid = labels.reshape(-1) != -100
        return -(lp.float().reshape(-1) * valid).sum(), valid.sum()

    def forward_only(self, input_ids, *, position_ids=None, cu_seqlens=None) -> torch.Tensor:
        """Final normalised hidden states (no gradients, parameters gathered unit by unit)."""
        model = self.model
        root, layers = self._units_by_role()
        self.gather(root)
        self.wait_gather(root)
        ctx = model.make_context(input_ids, position_ids, cu_seqlens, training=False)
        acts = model.forward_embed(input_ids, ctx)
        for i, unit in enumerate(layers):
            self.gather(unit)
            self.wait_gather(unit)
            if i + 1 < len(layers):
                self.gather(layers[i + 1])
            acts = unit.modules[0](*acts, ctx)
            if self.reshard:
                self.release(unit)
        hidden = model.forward_head(*acts, ctx)
        if self.reshard:
            self.release(root)
        return hidden

    # ---------------------------------------------------------------------------------------
    # gradient norm / clipping
    # ---------------------------------------------------------------------------------------
    def all_groups(self) -> Iterable[FlatParamGroup]:
        for u in self.units:
            yield from u.groups

    def grad_norm_and_clip_coef(self, max_norm: float) -> Tuple[torch.Tensor, torch.Tensor]:
        """Global L2 norm of the accumulated gradients and ``min(1, max_norm/(norm+1e-6))``, both as
        1-element device tensors (no host sync).  Dense shards are summed over the shard group,
        expert shards over ep_fsdp x ep (src/xorl/distributed/fsdp2/clip_grad_norm.py:60-257)."""
        dev = self.device
        dense_sq = torch.zeros(1, device=dev, dtype=torch.float32)
        expert_sq = torch.zeros(1, device=dev, dtype=torch.float32)
        first_d = first_e = True

        def counts_as_expert(g) -> bool:
            return getattr(g, "is_expert", False) and self.ps.ep_size > 1

        # lm-head rows under lm-head-only tensor parallelism: distinct rows on the ranks of an lm_head_tp group,
        # each sharded over its lm_head_replica group
        head_sq = torch.zeros(1, device=dev, dtype=torch.float32)
        head_groups = [g for g in self.all_groups() if getattr(g, "is_head", False) and g.grad_ready]
        for g in head_groups:
            head_sq += g.grad_shard.float().pow(2).sum()
            g.sq_valid = False

        if self.is_cuda:
            # per-unit partial sums taken early live on the side streams
            torch.cuda.current_stream().wait_stream(self.norm_stream)
            torch.cuda.current_stream().wait_stream(self.comm_stream)
        early_d, early_e = [], []
        for g in self.all_groups():
            if not g.grad_ready or getattr(g, "is_head", False):
                continue
            if g.sq_valid:
                (early_e if counts_as_expert(g) else early_d).append(g.sq)
                g.sq_valid = False
            elif counts_as_expert(g):
                optim_ops.sumsq_(g.grad_shard, expert_sq, not first_e)
                first_e = False
            else:
                optim_ops.sumsq_(g.grad_shard, dense_sq, not first_d)
                first_d = False
        # fixed order (unit order), one reduction: the same bits every run
        if early_d:
            dense_sq = dense_sq + torch.cat(early_d).sum()
        if early_e:
            expert_sq = expert_sq + torch.cat(early_e).sum()
        tp_pg = self.ps.group("tp") if self.ps.tp_size > 1 else None
        if tp_pg is not None:
            # replicated parameters (norm weights, embeddings) hold identical gradients on every
            # TP rank: count them once, sum only the tensor-parallel shards over the TP group.
            # Expert groups under expert parallelism are not part of dense_sq (they went into
            # expert_sq above) and are not sliced over the TP group, so they stay out of this split.
            rep_sq = torch.zeros(1, device=dev, dtype=torch.float32)
            for g in self.all_groups():
                if not g.grad_ready or counts_as_expert(g):
                    continue
                for i, a, b in g.param_segments_in_shard():
                    if getattr(g.named_params[i][1], "_xb_tp", None) is None:
                        rep_sq += g.grad_shard[a:b].float().pow(2).sum()
            sharded = (dense_sq - rep_sq).clamp_(min=0.0)
            dist.all_reduce(sharded, group=tp_pg)
            dense_sq = sharded + rep_sq
        if self.shard_pg is not None:
            dist.all_reduce(dense_sq, group=self.shard_pg)
        if self.ps.ep_size > 1:
            if self.ep_shard_pg is not None:
                dist.all_reduce(expert_sq, group=self.ep_shard_pg)
            if self.ps.group("ep") is not None:
                dist.all_reduce(expert_sq, group=self.ps.group("ep"))
        total = dense_sq + expert_sq
        if getattr(self.ps, "lm_head_tp_size", 1) > 1:
            if head_groups and head_groups[0].pg is not None:
                dist.all_reduce(head_sq, group=head_groups[0].pg)
            if self.ps.group("lm_head_tp") is not None:
                dist.all_reduce(head_sq, group=self.ps.group("lm_head_tp"))
            total = total + head_sq
        if self.ps.pp_size > 1 and self.ps.group("pp") is not None:
            dist.all_reduce(total, group=self.ps.group("pp"))
        norm = torch.zeros(1, device=dev, dtype=torch.float32)
        coef = torch.ones(1, device=dev, dtype=torch.float32)
        optim_ops.clip_coef_(total, max_norm, norm, coef)
        return norm, coef

    # ---------------------------------------------------------------------------------------
    # full-tensor access (checkpointing, export, weight sync)
    # ---------------------------------------------------------------------------------------
    @torch.no_grad()
    def iter_full_tensors(self, what: str = "master", extra: Optional[Dict[int, torch.Tensor]] = None,
                          ep_full: bool = True):
        """Yields (fqn, full tensor) unit by unit.  Expert-parallel parameters come back with all
        ``E`` experts (gathered over the ep group) unless ``ep_full`` is False, in which case they
        keep this rank's ``[E / ep, ...]`` rows.  ``what``: "master" (fp32 weights),
        "grad" (fp32 accumulated gradient) or "extra" with a {id(group): shard tensor} mapping
        (optimizer moments).  Every rank of the shard group must iterate in lock-step."""
        self.sync_optimizer()
        for g in self.all_groups():
            if what == "master":
                shard = g.master if g.master is not None else g.shard_lp
            elif getattr(g, "frozen", False):
                continue
            elif what == "grad":
                shard = g.grad_shard
            else:
                shard = extra[id(g)]
            if g.world > 1:
                full = torch.empty(g.padded, device=self.device, dtype=shard.dtype)
                dist.all_gather_into_tensor(full, shard.contiguous(), group=g.pg)
            else:
                full = shard
            for (name, p), view in zip(g.named_params, g.param_views(full)):
                spec = getattr(p, "_xb_tp", None)
                if spec is not None and self.ps.tp_size > 1:
                    from .tp import unshard_rows
                    parts = [torch.empty_like(view) for _ in range(self.ps.tp_size)]
                    dist.all_gather(parts, view.contiguous(), group=self.ps.group("tp"))
                    view = unshard_rows(parts, spec[1]) if spec[0] == "col" else torch.cat(parts, 1)
                if getattr(p, "_xb_lmtp", None) is not None and self.ps.group("lm_head_tp") is not None:
                    parts = [torch.empty_like(view) for _ in range(p._xb_lmtp[1])]
                    dist.all_gather(parts, view.contiguous(), group=self.ps.group("lm_head_tp"))
                    view = torch.cat(parts, 0)
                if ep_full and getattr(p, "_xb_ep", None) is not None and self.ps.ep_size > 1:
                    parts = [torch.empty_like(view) for _ in range(self.ps.ep_size)]
                    dist.all_gather(parts, view.contiguous(), group=self.ps.group("ep"))
                    view = torch.cat(parts, 0)
                yield name, view

    @torch.no_grad()
    def load_full_tensors(self, tensors: Dict[str, torch.Tensor], strict: bool = True,
                          target: str = "master", extra: Optional[Dict[int, torch.Tensor]] = None) -> List[str]:
        """Copies full tensors (by FQN) into this rank's shards.  Returns the missing names."""
        missing = []
        self.sync_optimizer()
        if target == "master":
            from ..ops.fp8_grouped import invalidate_weight_cache
            invalidate_weight_cache()
        for g in self.all_groups():
            if target != "master" and getattr(g, "frozen", False):
                continue
            dst = (g.master if g.master is not None else g.shard_lp) if target == "master" else extra[id(g)]
            s0, _ = g.shard_range()
            for i, a, b in g.param_segments_in_shard():
                name = g.named_params[i][0]
                if name not in tensors:
                    missing.append(name)
                    continue
                src = tensors[name]
                tp_slice = _slice_fn(g.named_params[i][1])
                if tp_slice is not None and tuple(src.shape) == tuple(g.named_params[i][1]._xb_full_shape):
                    src = tp_slice(src)
                src = src.reshape(-1)
                o = g.offsets[i]
                dst[a:b].copy_(src[s0 + a - o: s0 + b - o].to(device=self.device, dtype=dst.dtype))
            if target == "master":
                self.refresh_compute_copy(g)
        if strict and missing:
            raise KeyError(f"missing tensors: {sorted(set(missing))[:8]}")
        return sorted(set(missing))

    def refresh_compute_copy(self, g: FlatParamGroup) -> None:
        if g.master is not None and g.shard_lp is not g.master:
            g.shard_lp.copy_(g.master)

    def num_local_elements(self) -> int:
        return sum(g.shard_numel for g in self.all_groups())
