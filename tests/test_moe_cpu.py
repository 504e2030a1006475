"""MoE block on CPU: routing, aligned permutation, grouped MLP against a per-token loop."""
import torch

from xorl_b200.models.config import preset
from xorl_b200.models.context import StepContext
from xorl_b200.ops import moe as moe_ops
from xorl_b200.parallel.state import init_parallel_state, reset_parallel_state


def test_aligned_sort_indices():
    ids = torch.tensor([3, 0, 3, 1, 0, 3])
    dest, seg, counts = moe_ops.aligned_sort_indices(ids, 4, align=4)
    assert seg.tolist() == [0, 4, 8, 8, 12]
    assert counts.tolist() == [2, 1, 0, 3]
    assert dest.tolist() == [8, 0, 9, 4, 1, 10]


def test_moe_block_matches_naive():
    reset_parallel_state()
    init_parallel_state(device_type="cpu")
    from xorl_b200.models.moe import MoEBlock
    cfg = preset("qwen3-30b-a3b", hidden_size=64, num_experts=8, num_experts_per_tok=2,
                 moe_intermediate_size=32, num_hidden_layers=1)
    torch.manual_seed(0)
    blk = MoEBlock(cfg, 0, dtype=torch.float32)
    for p in blk.parameters():
        torch.nn.init.normal_(p, 0, 0.1)
    x = torch.randn(37, 64, requires_grad=True)
    ctx = StepContext(cu_seqlens=torch.tensor([0, 37], dtype=torch.int32), position_ids=torch.arange(37))
    ctx.aux["aux_loss_scale"] = 1.0
    out = blk(x, ctx)
    w, idx, probs = blk.gate(x)
    ref = torch.zeros_like(out)
    for t in range(37):
        for j in range(2):
            e = idx[t, j].item()
            h = x[t] @ blk.experts.gate_up_proj[e]
            a = torch.nn.functional.silu(h[:32]) * h[32:]
            ref[t] += w[t, j] * (a @ blk.experts.down_proj[e])
    assert torch.allclose(out, ref, atol=1e-5)
    aux = ctx.aux[("aux_loss", 0)]
    (out.sum() + aux).backward()
    assert x.grad is not None and blk.gate.weight.grad is not None
    assert blk.experts.gate_up_proj.grad.abs().sum() > 0


def test_canonical_combine_is_order_independent_and_exact():
    import torch
    from xorl_b200.ops.moe import canonical_combine
    torch.manual_seed(0)
    T, k, H = 7, 6, 9
    y = torch.randn(T, k, H).bfloat16()
    w = torch.rand(T, k)
    out = canonical_combine(y, w)
    ref = (y.double() * w.double().unsqueeze(-1))
    tree = ((ref[:, 0] + ref[:, 1]) + (ref[:, 2] + ref[:, 3])) + (ref[:, 4] + ref[:, 5])
    assert torch.equal(out, tree.to(torch.bfloat16))
    # the same bits whatever the memory layout of the slots (transposed storage, non-contiguous)
    y2 = y.permute(1, 0, 2).contiguous().permute(1, 0, 2)
    assert torch.equal(canonical_combine(y2, w), out)
