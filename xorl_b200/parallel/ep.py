"""Expert parallelism: token dispatch to the ranks that own the routed experts and combine back.

Two transports with the same semantics:

* ``alltoall`` — count exchange, ``all_to_all_single`` with variable splits (host-side split sizes),
  reorder by local expert, grouped expert MLP, reverse path.  This is the reference's baseline
  (src/xorl/distributed/moe/alltoall.py:44-362) and the CPU/gloo lane.
* ``fused`` — peer-memory path (``csrc/ep.cu``): every rank publishes its per-expert counts to all
  peers, computes every destination row on the device (no host sync), pushes token rows straight
  into the owners' segment-aligned receive buffers with peer stores, and the owners push expert
  outputs back to the source slots the same way.  Replaces DeepEP
  (src/xorl/distributed/moe/deepep.py:454-791).

In both, the weighted sum over the k experts of a token runs on the source rank in fp32.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import moe as moe_ops
from .state import get_parallel_state


def mark_ep(p: torch.nn.Parameter, ep_rank: int, ep_size: int) -> None:
    """Declares ``p`` (first dimension = local experts) as rows ``[ep_rank * n, (ep_rank + 1) * n)`` of
    a stacked ``[E, ...]`` tensor.  Initialisation draws the full tensor and keeps this slice, full
    tensors handed to ``Zero3Engine.load_full_tensors`` are sliced the same way, and checkpoints
    present the parameter as ``[Shard(0) over ep, Shard(1) over ep_fsdp]`` of the full shape
    (src/xorl/distributed/parallel_plan.py:331-393, src/xorl/checkpoint/checkpointer.py:107-160)."""
    n = p.shape[0]
    p._xb_ep = (int(ep_rank), int(ep_size))
    p._xb_full_shape = (n * ep_size, *p.shape[1:])
    p._xb_ep_slice = lambda full, a=ep_rank * n, b=(ep_rank + 1) * n: full[a:b]


class _AllToAll(torch.autograd.Function):
    """all_to_all_single with variable splits; backward is the reverse exchange."""

    @staticmethod
    def forward(ctx, x, out_splits: List[int], in_splits: List[int], group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits),) + tuple(x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), out_splits, in_splits, group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits),) + tuple(g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), ctx.in_splits, ctx.out_splits, group=ctx.group)
        return out, None, None, None


def _alltoall_forward(x, weights, indices, experts, num_experts, ctx):
    ps = get_parallel_state()
    group = ps.group("ep")
    ep = ps.ep_size
    El = num_experts // ep
    T, H = x.shape
    k = indices.shape[1]
    flat_e = indices.reshape(-1)
    # slots sorted by global expert id == sorted by (destination rank, local expert)
    order = torch.argsort(flat_e, stable=True)
    token_of_slot = torch.arange(T, device=x.device).repeat_interleave(k)
    send = x.index_select(0, token_of_slot.index_select(0, order))
    counts = torch.bincount(flat_e, minlength=num_experts)                     # [E]
    recv_counts = torch.empty_like(counts)
    dist.all_to_all_single(recv_counts, counts, group=group)                   # [ep * El] by source
    # split sizes must be host integers for the collective (the fused path avoids this sync)
    in_splits = counts.reshape(ep, El).sum(1).tolist()
    rc = recv_counts.reshape(ep, El)
    out_splits = rc.sum(1).tolist()
    recv = _AllToAll.apply(send, out_splits, in_splits, group)                 # grouped by source
    # received rows are ordered (source, local expert); build expert-major aligned segments
    src_ids = torch.repeat_interleave(torch.arange(ep, device=x.device), rc.sum(1))
    local_e = torch.repeat_interleave(torch.arange(El, device=x.device).repeat(ep), rc.reshape(-1))
    dest, seg, _ = moe_ops.aligned_sort_indices(local_e, El)
    rows = moe_ops.buffer_rows(recv.shape[0], El)
    buf = recv.new_zeros((rows, H)).index_copy(0, dest, recv)
    y = moe_ops.expert_mlp_aligned(buf, seg, experts.gate_up_proj, experts.down_proj,
                                   **moe_ops.experts_mlp_kwargs(experts))
    back = y.index_select(0, dest)
    ret = _AllToAll.apply(back, in_splits, out_splits, group)                  # sorted-slot order
    y_slots = _unsort(ret, order)
    if ctx.aux.get("canonical_moe", False):
        # parity lane: every token's k expert outputs are back on its own rank in the router's slot
        # order, so the fp64 fixed-tree combine gives the bits of the single-process result whatever
        # rank computed which expert (src/xorl/distributed/canonical_moe.py, deepep_canonical.py)
        return moe_ops.canonical_combine(y_slots.reshape(T, k, H), weights)
    out = (y_slots.reshape(T, k, H).float() * weights.unsqueeze(-1).float()).sum(1)
    return out.to(x.dtype)


def _unsort(sorted_rows: torch.Tensor, order: torch.Tensor) -> torch.Tensor:
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    return sorted_rows.index_select(0, inv)


def ep_moe_forward(x: torch.Tensor, weights: torch.Tensor, indices: torch.Tensor, experts,
                   num_experts: int, ctx) -> torch.Tensor:
    mode = ctx.aux.get("ep_dispatch", "alltoall")
    if ctx.aux.get("canonical_moe", False):
        mode = "alltoall"                 # the canonical combine lives on the all-to-all path
    if mode in ("fused", "deepep") and x.is_cuda and x.dtype == torch.bfloat16 \
            and ctx.aux.get("ep_workspace_reuse_ok", True):
        from .ep_fused import fused_ep_forward, fused_ep_available
        if fused_ep_available():
            return fused_ep_forward(x, weights, indices, experts, num_experts, ctx)
    return _alltoall_forward(x, weights, indices, experts, num_experts, ctx)
