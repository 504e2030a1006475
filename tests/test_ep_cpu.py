"""Expert parallelism over gloo: EP=2 dispatch/combine equals the all-local computation."""
import json
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _worker():
    import torch.distributed as dist
    from xorl_b200.models.config import preset
    from xorl_b200.models.context import StepContext
    from xorl_b200.models.moe import MoEBlock
    from xorl_b200.ops import moe as moe_ops
    from xorl_b200.parallel.state import init_parallel_state
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    init_parallel_state(device_type="cpu", ep_size=world)
    cfg = preset("qwen3-30b-a3b", hidden_size=32, num_experts=8, num_experts_per_tok=2,
                 moe_intermediate_size=16, num_hidden_layers=1)
    g = torch.Generator().manual_seed(0)
    full_gu = torch.randn(8, 32, 32, generator=g) * 0.2
    full_dn = torch.randn(8, 16, 32, generator=g) * 0.2
    gate_w = torch.randn(8, 32, generator=g) * 0.5
    blk = MoEBlock(cfg, 0, dtype=torch.float32)
    El = 8 // world
    with torch.no_grad():
        blk.gate.weight.copy_(gate_w)
        blk.experts.gate_up_proj.copy_(full_gu[rank * El:(rank + 1) * El])
        blk.experts.down_proj.copy_(full_dn[rank * El:(rank + 1) * El])
    gx = torch.Generator().manual_seed(10 + rank)
    x = torch.randn(19 + 3 * rank, 32, generator=gx, requires_grad=True)
    ctx = StepContext(cu_seqlens=torch.tensor([0, x.shape[0]], dtype=torch.int32),
                      position_ids=torch.arange(x.shape[0]))
    out = blk(x, ctx)
    out.square().sum().backward()
    # all-local oracle with the full expert tensors

    class E:  # noqa
        gate_up_proj = full_gu.clone().requires_grad_()
        down_proj = full_dn.clone().requires_grad_()
    xr = x.detach().clone().requires_grad_()
    w, idx, _ = blk.gate(xr)
    ref = moe_ops.local_moe_forward(xr, w, idx, E, 8)
    ref.square().sum().backward()
    ok = torch.allclose(out, ref, atol=1e-5) and torch.allclose(x.grad, xr.grad, atol=1e-4)
    # expert weight grads: sum of the oracle grads over ranks equals what the owner accumulated
    gsum = E.gate_up_proj.grad.clone()
    dist.all_reduce(gsum)
    ok = ok and torch.allclose(blk.experts.gate_up_proj.grad, gsum[rank * El:(rank + 1) * El], atol=1e-4)
    # canonical lane: the fp64 fixed-tree combine under expert parallelism gives the single-process
    # canonical result (the per-row expert outputs agree to fp32 rounding of the host GEMMs)
    ctx.aux["canonical_moe"] = True
    with torch.no_grad():
        can = blk(x.detach(), ctx)
        can_ref = moe_ops.local_moe_forward(x.detach(), w.detach(), idx, E, 8, canonical=True)
    ok = ok and torch.allclose(can, can_ref, atol=2e-6, rtol=0)
    flag = torch.tensor([1.0 if ok else 0.0])
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("EPOK " + json.dumps(bool(flag.item())))
    dist.destroy_process_group()


@pytest.mark.distributed
def test_ep_alltoall_matches_local():
    from dist_utils import run_distributed
    out = run_distributed(__file__, 2)
    assert "EPOK true" in out, out[-2000:]


if __name__ == "__main__":
    _worker()
