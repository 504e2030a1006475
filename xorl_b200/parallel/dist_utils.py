"""Small distributed helpers shared by the trainer and the service worker.

* ``token_normalised_loss`` -- a loss that is a sum over local tokens divided by the global token
  count, with the matching backward (src/xorl/distributed/gradient_accumulate_loss.py:7-64).
* ``synchronize_micro_batch_padding`` -- pad every rank's micro-batch to the widest one of the
  group by growing the trailing padding document (src/xorl/distributed/sync_padding.py:38-146; not
  applied under context parallelism).  No collective of this package needs equal shapes (flat
  parameter shards, capacity-sized expert workspaces, negotiated pipeline messages), so the trainer
  applies it only on request (``XORL_B200_SYNC_PADDING=1``), to equalise per-rank work.
* ``stochastic_bf16_all_to_all_reduce_scatter`` -- gradient reduce-scatter with bf16 on the wire:
  each rank rounds its fp32 gradient stochastically to bf16, exchanges slices with all-to-all and
  sums the received slices in fp32 (src/xorl/distributed/fsdp2/bf16_a2a_reduce.py:64-114).

Gradients of parameters that the reference replicates over the expert-parallel group (router, norms,
attention: src/xorl/distributed/ep_gradients.py) need no extra all-reduce here: every non-expert
parameter is ZeRO-sharded over all data ranks, so its reduce-scatter already sums over them.
"""
from __future__ import annotations

from typing import Dict, Iterable, List, Optional

import torch
import torch.distributed as dist

IGNORE_INDEX = -100


class _TokenNormalisedLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, loss_mean, local_tokens, group):
        t = torch.stack([loss_mean.detach().float() * local_tokens, local_tokens.float()])
        if group is not None and dist.is_initialized():
            dist.all_reduce(t, group=group)
        ctx.scale = (local_tokens.float() / t[1].clamp_min(1)).item() if t[1] > 0 else 0.0
        ctx.world = dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1
        return (t[0] / t[1].clamp_min(1)).to(loss_mean.dtype)

    @staticmethod
    def backward(ctx, g):
        # d(global mean)/d(local mean) = local_tokens / global_tokens; data-parallel gradient
        # averaging divides by the world size afterwards, so undo it here
        return g * ctx.scale * ctx.world, None, None


def token_normalised_loss(loss_mean: torch.Tensor, local_tokens: torch.Tensor, group=None) -> torch.Tensor:
    """``loss_mean`` is the mean over this rank's valid tokens; returns the mean over all ranks'
    valid tokens.  Use when the reducer averages gradients over ranks (DDP-style); the ZeRO engine
    itself sums gradients and takes ``grad_scale = 1 / global_tokens`` instead."""
    return _TokenNormalisedLoss.apply(loss_mean, local_tokens, group)


def synchronize_micro_batch_padding(micro_batches: List[Dict[str, torch.Tensor]], group=None,
                                    pad_token_id: int = 0, multiple_of: int = 1) -> List[Dict[str, torch.Tensor]]:
    """Pads micro-batch i of every rank to the group's maximum length of micro-batch i."""
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return micro_batches
    lens = torch.tensor([mb["input_ids"].shape[-1] for mb in micro_batches], dtype=torch.long)
    dev = "cuda" if dist.get_backend(group) == "nccl" else "cpu"
    lens = lens.to(dev)
    dist.all_reduce(lens, op=dist.ReduceOp.MAX, group=group)
    out = []
    for mb, target in zip(micro_batches, lens.tolist()):
        target = (target + multiple_of - 1) // multiple_of * multiple_of
        T = mb["input_ids"].shape[-1]
        if target == T:
            out.append(mb)
            continue
        pad = target - T
        nb = dict(mb)

        def grow(t, value):
            shape = list(t.shape)
            shape[-1] = pad
            return torch.cat([t, torch.full(shape, value, dtype=t.dtype, device=t.device)], -1)

        nb["input_ids"] = grow(mb["input_ids"], pad_token_id)
        nb["labels"] = grow(mb["labels"], IGNORE_INDEX)
        if "position_ids" in mb:
            extra = torch.arange(pad, dtype=mb["position_ids"].dtype, device=mb["position_ids"].device)
            nb["position_ids"] = torch.cat([mb["position_ids"], extra.expand(*mb["position_ids"].shape[:-1], pad)], -1)
        if "cu_seqlens" in mb:
            cu = mb["cu_seqlens"]
            nb["cu_seqlens"] = torch.cat([cu, cu[-1:] + pad])     # the padding is one more document
        out.append(nb)
    return out


def stochastic_round_bf16(x: torch.Tensor, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """fp32 -> bf16 rounding up or down with probability proportional to the distance."""
    if x.is_cuda:
        from ..ops import optim as optim_ops
        if hasattr(optim_ops, "stochastic_round_bf16"):
            return optim_ops.stochastic_round_bf16(x)
    bits = x.contiguous().view(torch.int32)
    noise = torch.randint(0, 1 << 16, bits.shape, dtype=torch.int32, device=x.device, generator=generator)
    return ((bits + noise) & ~0xFFFF).view(torch.float32).to(torch.bfloat16)


def stochastic_bf16_all_to_all_reduce_scatter(grad: torch.Tensor, out_shard: torch.Tensor, group,
                                              accumulate: bool = False) -> None:
    """``grad`` fp32 [world * n]; ``out_shard`` fp32 [n] receives (or accumulates) the sum over
    ranks of slice [rank].  bf16 on the wire, fp32 summation in a fixed rank order."""
    world = dist.get_world_size(group)
    n = out_shard.numel()
    send = stochastic_round_bf16(grad).view(world, n)
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv.view(-1), send.view(-1), group=group)
    total = recv.float().sum(0)
    if accumulate:
        out_shard.add_(total)
    else:
        out_shard.copy_(total)
