"""Global parallel state: one N-D rank grid ``[pp, dp_replicate, dp_shard, ringattn, ulysses, tp]``
plus the expert-parallel grid ``[pp, ep_fsdp, ep]`` and the lm-head TP grid, each dimension with
its own process group.

Same dimension order, flattened aliases (``dp``, ``sp``, ``dp_shard_sp``, ``dp_sp``) and
``cp_fsdp_mode`` folding rules as the reference (src/xorl/distributed/parallel_state.py:119-138,
625-851), built directly on ``torch.distributed.new_group`` so that it also runs over gloo on CPU.
"""
from __future__ import annotations

import itertools
import os
from dataclasses import dataclass, field
from datetime import timedelta
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

DIM_NAMES = ("pp", "dp_replicate", "dp_shard", "ringattn", "ulysses", "tp")


def process_group_timeout() -> timedelta:
    """XORL_PROCESS_GROUP_TIMEOUT_MINUTES, default 60, minimum 1 (src/xorl/utils/device.py:25-51)."""
    raw = os.environ.get("XORL_PROCESS_GROUP_TIMEOUT_MINUTES", "60")
    try:
        minutes = max(1.0, float(raw))
    except ValueError:
        minutes = 60.0
    return timedelta(minutes=minutes)


class _Group:
    """A process group together with its ranks; size-1 groups carry no torch group."""

    def __init__(self, ranks: Sequence[int], pg):
        self.ranks = list(ranks)
        self.pg = pg

    @property
    def size(self) -> int:
        return len(self.ranks)

    def rank_in_group(self, global_rank: int) -> int:
        return self.ranks.index(global_rank)


@dataclass
class ParallelState:
    world_size: int = 1
    rank: int = 0
    device_type: str = "cpu"
    sizes: Dict[str, int] = field(default_factory=lambda: {n: 1 for n in DIM_NAMES})
    coords: Dict[str, int] = field(default_factory=lambda: {n: 0 for n in DIM_NAMES})
    groups: Dict[str, _Group] = field(default_factory=dict)
    ep_size: int = 1
    ep_fsdp_size: int = 1
    lm_head_tp_size: int = 1
    dp_mode: str = "fsdp2"
    cp_fsdp_mode: str = "all"
    tp_sequence_parallel: bool = False   # residual stream sharded by tokens between TP regions

    # ---- sizes ------------------------------------------------------------------------------
    def size(self, name: str) -> int:
        if name in self.sizes:
            return self.sizes[name]
        return self.groups[name].size if name in self.groups else 1

    @property
    def pp_size(self): return self.sizes["pp"]
    @property
    def tp_size(self): return self.sizes["tp"]
    @property
    def ulysses_size(self): return self.sizes["ulysses"]
    @property
    def ringattn_size(self): return self.sizes["ringattn"]
    @property
    def sp_size(self): return self.sizes["ulysses"] * self.sizes["ringattn"]
    @property
    def dp_shard_size(self): return self.sizes["dp_shard"]
    @property
    def dp_replicate_size(self): return self.sizes["dp_replicate"]
    @property
    def dp_size(self): return self.sizes["dp_shard"] * self.sizes["dp_replicate"]

    # ---- ranks ------------------------------------------------------------------------------
    def rank_in(self, name: str) -> int:
        g = self.groups.get(name)
        return g.rank_in_group(self.rank) if g is not None else 0

    @property
    def pp_rank(self): return self.coords["pp"]
    @property
    def tp_rank(self): return self.coords["tp"]
    @property
    def dp_rank(self): return self.rank_in("dp")
    @property
    def ep_rank(self): return self.rank_in("ep")
    @property
    def sp_rank(self): return self.rank_in("sp")
    @property
    def ulysses_rank(self): return self.coords["ulysses"]
    @property
    def ringattn_rank(self): return self.coords["ringattn"]

    def group(self, name: str):
        """torch ProcessGroup (None for a singleton group)."""
        g = self.groups.get(name)
        return g.pg if g is not None else None

    def group_ranks(self, name: str) -> List[int]:
        g = self.groups.get(name)
        return list(g.ranks) if g is not None else [self.rank]

    # ---- semantic aliases ---------------------------------------------------------------------
    @property
    def fsdp_group_name(self) -> str:
        """Group over which dense parameters are ZeRO-sharded: dp_shard folded with the SP ranks
        selected by cp_fsdp_mode (src/xorl/distributed/parallel_state.py:349-366)."""
        return "fsdp"

    @property
    def loss_group_name(self) -> str:
        """Token counts / losses are normalised over dp x sp."""
        return "dp_sp"


_STATE: Optional[ParallelState] = None


def get_parallel_state() -> ParallelState:
    global _STATE
    if _STATE is None:
        _STATE = ParallelState()
    return _STATE


def reset_parallel_state() -> None:
    global _STATE
    _STATE = None


def _make_groups(all_rank_lists: List[List[int]], my_rank: int, backend) -> Optional[_Group]:
    """Every rank must create every group of a family, in the same order."""
    mine = None
    for ranks in all_rank_lists:
        pg = dist.new_group(ranks=ranks, backend=backend, timeout=process_group_timeout()) \
            if len(ranks) > 1 else None
        if my_rank in ranks:
            mine = _Group(ranks, pg)
    return mine


def init_parallel_state(*, dp_size: int = -1, dp_replicate_size: int = 1, dp_shard_size: int = -1,
                        tp_size: int = 1, ep_size: int = 1, pp_size: int = 1, ulysses_size: int = 1,
                        ringattn_size: int = 1, lm_head_tp_size: int = 1, dp_mode: str = "fsdp2",
                        cp_fsdp_mode: str = "all", device_type: Optional[str] = None,
                        ep_intranode: bool = True, tp_sequence_parallel: bool = False) -> ParallelState:
    """Builds every process group.  ``torch.distributed`` must be initialised when world > 1."""
    global _STATE
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    if device_type is None:
        device_type = "cuda" if torch.cuda.is_available() else "cpu"
    non_dp = pp_size * tp_size * ulysses_size * ringattn_size
    if world % non_dp:
        raise ValueError(f"world size {world} not divisible by pp*tp*ulysses*ringattn={non_dp}")
    dp = world // non_dp
    if dp_size not in (-1, dp):
        raise ValueError(f"dp_size {dp_size} inconsistent with world size {world} (expected {dp})")
    if dp_shard_size <= 0:
        dp_shard_size = dp // max(1, dp_replicate_size)
    if dp_replicate_size <= 0:
        dp_replicate_size = dp // dp_shard_size
    if dp_replicate_size * dp_shard_size != dp:
        raise ValueError(f"dp_replicate ({dp_replicate_size}) x dp_shard ({dp_shard_size}) != dp ({dp})")
    sizes = {"pp": pp_size, "dp_replicate": dp_replicate_size, "dp_shard": dp_shard_size,
             "ringattn": ringattn_size, "ulysses": ulysses_size, "tp": tp_size}
    shape = [sizes[n] for n in DIM_NAMES]
    grid = torch.arange(world).reshape(shape)
    my = (grid == rank).nonzero()[0].tolist()
    coords = {n: my[i] for i, n in enumerate(DIM_NAMES)}
    st = ParallelState(world_size=world, rank=rank, device_type=device_type, sizes=sizes,
                       coords=coords, ep_size=ep_size, lm_head_tp_size=lm_head_tp_size,
                       dp_mode=dp_mode, cp_fsdp_mode=cp_fsdp_mode,
                       tp_sequence_parallel=bool(tp_sequence_parallel and tp_size > 1))
    backend = None  # default backend of the world group

    def family(dims: Sequence[str]) -> List[List[int]]:
        """All groups obtained by varying `dims` (flattened in grid order) and fixing the rest."""
        idx = [DIM_NAMES.index(d) for d in dims]
        rest = [i for i in range(len(DIM_NAMES)) if i not in idx]
        perm = grid.permute(*rest, *idx).reshape(-1, int(torch.tensor([shape[i] for i in idx]).prod()))
        return [row.tolist() for row in perm]

    if world > 1:
        fsdp_dims = ["dp_shard"]
        if cp_fsdp_mode in ("all", "ring_only"):
            fsdp_dims.append("ringattn")
        if cp_fsdp_mode in ("all", "ulysses_only"):
            fsdp_dims.append("ulysses")
        sp_not_in_fsdp = [d for d in ("ringattn", "ulysses") if d not in fsdp_dims]
        families = {
            "pp": ["pp"], "tp": ["tp"], "ulysses": ["ulysses"], "ringattn": ["ringattn"],
            "dp_shard": ["dp_shard"], "dp_replicate": ["dp_replicate"],
            "dp": ["dp_replicate", "dp_shard"],
            "sp": ["ringattn", "ulysses"],
            "dp_sp": ["dp_replicate", "dp_shard", "ringattn", "ulysses"],
            "dp_shard_sp": ["dp_shard", "ringattn", "ulysses"],
            "fsdp": fsdp_dims,
            "stage": ["dp_replicate", "dp_shard", "ringattn", "ulysses", "tp"],
        }
        if sp_not_in_fsdp:
            families["sp_grad_sync"] = sp_not_in_fsdp
        for name, dims in families.items():
            g = _make_groups(family(dims), rank, backend)
            if g is not None:
                st.groups[name] = g
        # expert-parallel grid inside each pipeline stage: [ep_fsdp, ep], ep innermost (adjacent
        # ranks) when ep_intranode, outermost otherwise (src/xorl/distributed/parallel_state.py:739-757)
        ranks_per_stage = world // pp_size
        if ep_size > 1:
            if ranks_per_stage % ep_size:
                raise ValueError(f"ranks per stage {ranks_per_stage} not divisible by ep {ep_size}")
            ep_fsdp = ranks_per_stage // ep_size
            st.ep_fsdp_size = ep_fsdp
            ep_lists, epf_lists = [], []
            for s in range(pp_size):
                stage_ranks = grid[s].reshape(-1)
                g2 = stage_ranks.reshape(ep_fsdp, ep_size) if ep_intranode else \
                    stage_ranks.reshape(ep_size, ep_fsdp).t()
                ep_lists += [row.tolist() for row in g2]
                epf_lists += [col.tolist() for col in g2.t()]
            for name, lists in (("ep", ep_lists), ("ep_fsdp", epf_lists)):
                g = _make_groups(lists, rank, backend)
                if g is not None:
                    st.groups[name] = g
        if lm_head_tp_size > 1:
            if tp_size != 1:
                raise ValueError("lm_head_tp_size > 1 requires tp_size == 1")
            lists, rep_lists = [], []
            for s in range(pp_size):
                stage_ranks = grid[s].reshape(-1)
                g2 = stage_ranks.reshape(-1, lm_head_tp_size)
                lists += [row.tolist() for row in g2]
                rep_lists += [col.tolist() for col in g2.t()]
            for name, l in (("lm_head_tp", lists), ("lm_head_replica", rep_lists)):
                g = _make_groups(l, rank, backend)
                if g is not None:
                    st.groups[name] = g
    else:
        st.ep_fsdp_size = 1
    if ep_size > 1 and world == 1:
        raise ValueError("expert_parallel_size > 1 needs more than one rank")
    _STATE = st
    return st
