"""Tensor parallelism: column / row sharded linears with the matching collectives in autograd.

Column-parallel (``qkv_proj``, ``gate_up_proj``): the output features are split over the TP ranks
(section-wise for fused projections so that every rank holds whole q / k / v heads and matching
gate / up rows); the replicated input needs an all-reduce of its gradient.  Row-parallel
(``o_proj``, ``down_proj``): the input features are split and the partial outputs are summed.
Same plan as the reference's TP_PLAN (src/xorl/models/transformers/qwen3/parallelize.py:5-17,
src/xorl/distributed/torch_parallelize.py:222-270); per-head qk-norm weights see only local heads,
so their gradients are summed over the TP group before the optimizer step.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from .state import get_parallel_state


def tp_info():
    ps = get_parallel_state()
    return ps.tp_size, ps.tp_rank, ps.group("tp")


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_tp(x, group):
    return _CopyToTP.apply(x, group) if group is not None else x


def reduce_from_tp(x, group):
    return _ReduceFromTP.apply(x, group) if group is not None else x


def shard_rows(full: torch.Tensor, sections: Sequence[int], tp: int, rank: int) -> torch.Tensor:
    """Column-parallel weight [out, in]: every section of the output rows is split evenly."""
    parts = []
    off = 0
    for s in sections:
        per = s // tp
        parts.append(full[off + rank * per: off + (rank + 1) * per])
        off += s
    return torch.cat(parts, 0)


def shard_cols(full: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """Row-parallel weight [out, in]: input columns are split evenly."""
    per = full.shape[1] // tp
    return full[:, rank * per:(rank + 1) * per]


def unshard_rows(parts: List[torch.Tensor], sections: Sequence[int]) -> torch.Tensor:
    tp = len(parts)
    out = []
    off = [0] * tp
    for s in sections:
        per = s // tp
        for r in range(tp):
            out.append(parts[r][off[r]:off[r] + per])
            off[r] += per
    return torch.cat(out, 0)


def mark_col(p: torch.nn.Parameter, full_shape, sections: Sequence[int]) -> None:
    tp, rank, _ = tp_info()
    p._xb_tp = ("col", tuple(sections))
    p._xb_full_shape = tuple(full_shape)
    p._xb_tp_slice = lambda full, s=tuple(sections), t=tp, r=rank: shard_rows(full, s, t, r)


def mark_lm_head(p: torch.nn.Parameter, full_shape, size: int, rank: int) -> None:
    """``p`` holds vocabulary rows ``[rank * V / size, (rank + 1) * V / size)`` of the lm-head: lm-head-only
    tensor parallelism over the ``lm_head_tp`` group (consecutive data-parallel ranks).  ZeRO shards such
    a parameter over the ranks that hold the same rows (``lm_head_replica``)."""
    per = full_shape[0] // size
    p._xb_lmtp = (int(rank), int(size))
    p._xb_full_shape = tuple(full_shape)
    p._xb_lmtp_slice = lambda full, a=rank * per, b=(rank + 1) * per: full[a:b]


class _OwnShare(torch.autograd.Function):
    """Value ``x / size`` (every rank of the group computed the same group total: the shares add up to it
    over the group), gradient passed through unscaled (every rank back-propagates the whole total
    through its own vocabulary rows)."""

    @staticmethod
    def forward(ctx, x, size):
        return x / size

    @staticmethod
    def backward(ctx, g):
        return g, None


def mark_row(p: torch.nn.Parameter, full_shape) -> None:
    tp, rank, _ = tp_info()
    p._xb_tp = ("row", ())
    p._xb_full_shape = tuple(full_shape)
    p._xb_tp_slice = lambda full, t=tp, r=rank: shard_cols(full, t, r)
