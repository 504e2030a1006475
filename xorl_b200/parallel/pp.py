"""Pipeline-parallel runtime: stage assignment, point-to-point plumbing, schedule executor.

Each rank builds only its own layers (``assign_layers``), wraps them in a ZeRO engine (sharded over
the data-parallel ranks of the stage) and executes the action list of ``pp_schedules`` for every
optimizer step.  Activations cross stage boundaries as one ``[2, T, H]`` tensor (hidden, residual)
over NCCL / gloo send-recv, posted asynchronously so they overlap compute.  One process group per
ordered (sender -> receiver) pair keeps every communicator one-directional: messages are matched
in the sender's program order, which the receiver knows because all ranks hold all action lists.
Zero-bubble schedules split backward: ``I`` runs the backward with the weight-gradient GEMMs
captured (``grad_sink.defer_wgrad``), ``W`` runs them and reduces the gradients.

Reference: src/xorl/distributed/pipeline_parallel.py:138-789, src/xorl/trainers/training_utils.py:788-851.
"""
from __future__ import annotations

import os
import time
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import grad_sink
from . import pp_schedules as S
from .pp_contract import assert_wire_dtype, validate_microbatch_metadata
from .state import ParallelState, process_group_timeout


def assign_layers(num_layers: int, pp: int, schedule: str, virtual_stages: int = 1,
                  input_weight: int = 1, output_weight: int = 1,
                  first: Optional[int] = None, last: Optional[int] = None) -> List[List[int]]:
    """Layers of every global stage.  The embedding counts as ``input_weight`` layers of work on the
    first stage and the head as ``output_weight`` on the last when balancing
    (src/xorl/distributed/pipeline_parallel.py:164-334)."""
    n_stages = pp * S.num_chunks(schedule.lower(), virtual_stages)
    if n_stages > num_layers:
        raise ValueError(f"{n_stages} pipeline stages for only {num_layers} layers")
    counts = [0] * n_stages
    if first is not None or last is not None:
        f = first if first is not None else None
        l = last if last is not None else None
        rest = num_layers - (f or 0) - (l or 0)
        mid = n_stages - (f is not None) - (l is not None)
        base, extra = divmod(rest, max(mid, 1))
        k = 0
        for s in range(n_stages):
            if s == 0 and f is not None:
                counts[s] = f
            elif s == n_stages - 1 and l is not None:
                counts[s] = l
            else:
                counts[s] = base + (1 if k < extra else 0)
                k += 1
    else:
        total = num_layers + input_weight + output_weight
        per = total / n_stages
        remaining = num_layers
        for s in range(n_stages):
            w = per - (input_weight if s == 0 else 0) - (output_weight if s == n_stages - 1 else 0)
            counts[s] = max(1, round(w))
        # fix rounding drift while keeping every stage non-empty
        diff = num_layers - sum(counts)
        s = n_stages // 2
        while diff != 0:
            if diff > 0:
                counts[s % n_stages] += 1; diff -= 1
            elif counts[s % n_stages] > 1:
                counts[s % n_stages] -= 1; diff += 1
            s += 1
    out, cur = [], 0
    for c in counts:
        out.append(list(range(cur, cur + c)))
        cur += c
    assert cur == num_layers
    return out


def local_stage_layout(num_layers: int, ps: ParallelState, schedule: str, virtual_stages: int = 1,
                       **kw) -> Dict:
    """What this pipeline rank builds: the layers of each local chunk and embed / head ownership."""
    pp, r = ps.pp_size, ps.pp_rank
    sched = schedule.lower()
    stages = assign_layers(num_layers, pp, sched, virtual_stages, **kw)
    chunks = S.num_chunks(sched, virtual_stages)
    n_stages = pp * chunks
    local = [S.global_stage(r, c, pp, sched) for c in range(chunks)]
    layout = {"chunk_layers": [stages[g] for g in local], "chunk_stage": local, "n_stages": n_stages,
              "has_embed": 0 in local, "has_head": (n_stages - 1) in local,
              "layers": sorted(sum((stages[g] for g in local), []))}
    from .pp_contract import validate_layout, validate_stage_plan
    validate_stage_plan(stages, num_layers)
    validate_layout(layout, num_layers)
    return layout


class _PairGroups:
    """One process group per ordered pair of pipeline ranks that exchange messages."""

    def __init__(self, ps: ParallelState, pairs: List[Tuple[int, int]]):
        self.groups: Dict[Tuple[int, int], object] = {}
        pp_ranks_all = _all_pp_rank_lists(ps)
        for ranks in pp_ranks_all:               # every rank creates every group, same order
            for (a, b) in pairs:
                g = dist.new_group(ranks=[ranks[a], ranks[b]], timeout=process_group_timeout())
                if ps.rank in ranks:
                    self.groups[(a, b)] = g
        self.my_ranks = ps.group_ranks("pp")


def _all_pp_rank_lists(ps: ParallelState) -> List[List[int]]:
    world, pp = ps.world_size, ps.pp_size
    per = world // pp
    return [[s * per + i for s in range(pp)] for i in range(per)]


class PipelineRunner:
    def __init__(self, engine, ps: ParallelState, schedule: str, virtual_stages: int, layout: Dict,
                 n_microbatches: int):
        self.engine, self.ps = engine, ps
        self.schedule = schedule.lower()
        self.virtual_stages = virtual_stages
        self.bubble_stats: Dict[str, float] = {}
        self.pp, self.rank = ps.pp_size, ps.pp_rank
        self.layout = layout
        self.n_mb = n_microbatches
        self.chunks = len(layout["chunk_layers"])
        self.n_stages = layout["n_stages"]
        self.actions = S.build_schedule(self.schedule, self.pp, n_microbatches, virtual_stages)
        S.simulate(self.actions, self.schedule, self.pp, n_microbatches, virtual_stages)
        root, layer_units = engine._units_by_role()
        self.root = root
        by_name = {u.name: u for u in layer_units}
        self.chunk_units = [[by_name[f"layers.{i}"] for i in ls] for ls in layout["chunk_layers"]]
        pairs = set()
        for g in range(self.n_stages - 1):
            a, _ = S.stage_owner(g, self.pp, self.schedule)
            b, _ = S.stage_owner(g + 1, self.pp, self.schedule)
            if a != b:
                pairs.add((a, b))
                pairs.add((b, a))
        self.pairs = _PairGroups(ps, sorted(pairs)) if self.pp > 1 else None
        self._send_order = self._message_orders()

    # ---- message ordering -----------------------------------------------------------------------
    def _message_orders(self) -> Dict[Tuple[int, int], List[Tuple[str, int, int]]]:
        """For every ordered pair (src, dst): the messages in the order the source emits them.
        A message is (kind, microbatch, source global stage)."""
        order: Dict[Tuple[int, int], List] = {}
        for r in range(self.pp):
            for op, m, c in self.actions[r]:
                g = S.global_stage(r, c, self.pp, self.schedule)
                if op == "F" and g < self.n_stages - 1:
                    dst, _ = S.stage_owner(g + 1, self.pp, self.schedule)
                    if dst != r:
                        order.setdefault((r, dst), []).append(("F", m, g))
                elif op in ("B", "I") and g > 0:
                    dst, _ = S.stage_owner(g - 1, self.pp, self.schedule)
                    if dst != r:
                        order.setdefault((r, dst), []).append(("B", m, g))
        return order

    # ---- one optimizer step -----------------------------------------------------------------------
    def run(self, micro_batches: List[Dict[str, torch.Tensor]], grad_scale: float) -> torch.Tensor:
        eng = self.engine
        dev = eng.device
        assert len(micro_batches) == self.n_mb, (len(micro_batches), self.n_mb)
        # XORL_PP_BUBBLE_PROFILE=1: time spent waiting for a neighbour's activation or gradient,
        # against the whole step (the device is synchronised around each wait, so the profile
        # perturbs the run it measures; src/xorl/distributed/pp_profiling.py has the same switch)
        profile = os.environ.get("XORL_PP_BUBBLE_PROFILE", "0") == "1"
        prof = {"wait_s": 0.0, "waits": 0, "sent_bytes": 0}
        t_step = time.perf_counter()

        def _sync():
            if dev.type == "cuda":
                torch.cuda.synchronize()
        for i, mb in enumerate(micro_batches):
            if mb.get("cu_seqlens") is not None and mb.get("position_ids") is not None:
                validate_microbatch_metadata(mb, i)
        ctxs = [eng.make_step_context(mb["input_ids"], mb.get("position_ids"), mb.get("cu_seqlens"),
                                      grad_scale) for mb in micro_batches]
        H = eng.model.config.hidden_size
        dtype = eng.compute_dtype
        saved: Dict[Tuple[int, int], List] = {}
        outputs: Dict[Tuple[int, int], Tuple] = {}     # activations kept for a local next stage / head
        local_in: Dict[Tuple[str, int, int], torch.Tensor] = {}
        pending_w: Dict[Tuple[int, int], Tuple[List, List]] = {}
        posted: Dict[Tuple[int, int], int] = {}
        recv_bufs: Dict[Tuple[str, int, int], Tuple[torch.Tensor, object]] = {}
        sends: List = []
        loss_total = torch.zeros((), device=dev, dtype=torch.float32)
        if self.root is not None:
            eng.gather(self.root)
            eng.wait_gather(self.root)
            eng._prepare_grad_buffers(self.root)

        def pack(acts):
            h, res = acts
            t = torch.empty((2,) + tuple(h.shape), device=dev, dtype=dtype)
            t[0].copy_(h)
            if res is None:
                t[1].zero_()
            else:
                t[1].copy_(res)
            return t

        def send(kind, m, g, dst, tensor):
            assert_wire_dtype(tensor, dtype, f"{kind} of micro-batch {m} from stage {g}")
            grp = self.pairs.groups[(self.rank, dst)]
            w = dist.isend(tensor, dst=self.pairs.my_ranks[dst], group=grp)
            sends.append((w, tensor))
            prof["sent_bytes"] += tensor.numel() * tensor.element_size()

        def recv(kind, m, g, src, T):
            """Blocks until message (kind, m, g) from pipeline rank `src` has arrived; posts the
            receives of that pair in the sender's order up to and including this one."""
            key = (kind, m, g)
            seq = self._send_order[(src, self.rank)]
            grp = self.pairs.groups[(src, self.rank)]
            want = seq.index(key)
            nxt = posted.get((src, self.rank), 0)
            while nxt <= want:
                k2 = seq[nxt]
                Tk = ctxs[k2[1]].num_tokens
                buf = torch.empty((2, Tk, H), device=dev, dtype=dtype)
                w = dist.irecv(buf, src=self.pairs.my_ranks[src], group=grp)
                recv_bufs[k2] = (buf, w)
                nxt += 1
            posted[(src, self.rank)] = nxt
            buf, w = recv_bufs.pop(key)
            if profile:
                _sync()
                t0 = time.perf_counter()
                w.wait()
                _sync()
                prof["wait_s"] += time.perf_counter() - t0
                prof["waits"] += 1
            else:
                w.wait()
            return buf

        for op, m, c in self.actions[self.rank]:
            g = self.layout["chunk_stage"][c]
            ctx = ctxs[m]
            mb = micro_batches[m]
            units = self.chunk_units[c]
            if op == "F":
                if g == 0:
                    with torch.no_grad():
                        acts = eng.model.forward_embed(mb["input_ids"], ctx)
                else:
                    src, _ = S.stage_owner(g - 1, self.pp, self.schedule)
                    buf = local_in.pop(("F", m, g - 1)) if src == self.rank else \
                        recv("F", m, g - 1, src, ctx.num_tokens)
                    acts = (buf[0], buf[1])
                acts, sv = eng.chunk_forward(units, acts, ctx)
                saved[(m, c)] = sv
                if g == self.n_stages - 1:
                    outputs[(m, c)] = acts
                else:
                    dst, _ = S.stage_owner(g + 1, self.pp, self.schedule)
                    t = pack(acts)
                    if dst == self.rank:
                        local_in[("F", m, g)] = t
                    else:
                        send("F", m, g, dst, t)
            elif op in ("B", "I"):
                if g == self.n_stages - 1:
                    loss, dacts = eng.head_forward_backward(outputs.pop((m, c)), mb["labels"], ctx,
                                                            grad_scale)
                    loss_total = loss_total + loss
                else:
                    src, _ = S.stage_owner(g + 1, self.pp, self.schedule)
                    buf = local_in.pop(("B", m, g + 1)) if src == self.rank else \
                        recv("B", m, g + 1, src, ctx.num_tokens)
                    dacts = (buf[0], buf[1])
                if op == "I":
                    with grad_sink.defer_wgrad() as store:
                        dacts, pend = eng.chunk_backward(units, saved.pop((m, c)), dacts, ctx,
                                                         defer_reduce=True)
                    pending_w[(m, c)] = (store, pend)
                else:
                    dacts, _ = eng.chunk_backward(units, saved.pop((m, c)), dacts, ctx)
                if g == 0:
                    eng.embed_backward(mb["input_ids"], ctx, dacts)
                else:
                    dst, _ = S.stage_owner(g - 1, self.pp, self.schedule)
                    h, res = dacts
                    t = pack((h if h is not None else torch.zeros_like(res), res))
                    if dst == self.rank:
                        local_in[("B", m, g)] = t
                    else:
                        send("B", m, g, dst, t)
            else:  # W
                store, pend = pending_w.pop((m, c))
                for fn in store:
                    fn()
                eng.reduce_deferred(pend)
        for w, _t in sends:
            w.wait()
        if self.root is not None:
            eng._reduce_unit_grads(self.root)
            if eng.reshard:
                eng.release(self.root)
        # the loss lives on the last stage: share it along the pipeline group
        if self.pp > 1 and self.ps.group("pp") is not None:
            dist.all_reduce(loss_total, group=self.ps.group("pp"))
        if profile:
            _sync()
            step_s = time.perf_counter() - t_step
            self.bubble_stats = {
                "step_s": step_s, "wait_s": prof["wait_s"], "waits": prof["waits"],
                "measured_bubble_fraction": prof["wait_s"] / max(step_s, 1e-9),
                "analytic_bubble_fraction": S.analytic_bubble_fraction(self.schedule, self.pp, self.n_mb,
                                                                       self.virtual_stages),
                "p2p_sent_bytes": prof["sent_bytes"]}
        return loss_total
