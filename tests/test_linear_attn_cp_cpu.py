"""Context-parallel gated delta rule and short convolution on gloo ranks against the single-process
result (outputs and gradients), with documents that straddle, end at, and start inside shard borders."""
import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

T_LOCAL, H, DK, DV, C, K = 48, 2, 8, 6, 16, 4


def _inputs(world):
    torch.manual_seed(0)
    T = T_LOCAL * world
    f = lambda *s: torch.randn(*s, dtype=torch.float64)
    q = torch.nn.functional.normalize(f(T, H, DK), dim=-1)
    k = torch.nn.functional.normalize(f(T, H, DK), dim=-1)
    v, g, beta = f(T, H, DV), -torch.rand(T, H, dtype=torch.float64), torch.rand(T, H, dtype=torch.float64)
    x, w, b = f(T, C), f(C, K), f(C)
    # one document crosses the first border, one ends exactly on the second border (world 3),
    # the last 5 tokens are padding
    cu = sorted({0, 10, T_LOCAL + 7, 2 * T_LOCAL, T - 5})
    wo, wy = f(T, H, DV), f(T, C)
    return q, k, v, g, beta, x, w, b, torch.tensor(cu, dtype=torch.int32), wo, wy


def test_shard_documents():
    from xorl_b200.parallel.linear_attn_cp import shard_documents
    cu = [0, 10, 55, 96, 139]
    assert shard_documents(cu, 0, 48) == ([0, 10, 48], False)
    assert shard_documents(cu, 48, 96) == ([0, 7, 48], True)
    assert shard_documents(cu, 96, 144) == ([0, 43, 48], False)
    assert shard_documents(cu, 45, 96) == ([0, 10, 51], True)


def _worker():
    import torch.distributed as dist
    from xorl_b200.models.gated_deltanet import gated_delta_rule
    from xorl_b200.ops.seqmix import causal_conv1d_reference
    from xorl_b200.parallel.linear_attn_cp import causal_conv1d_cp, gated_delta_rule_cp
    import datetime
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    q, k, v, g, beta, x, w, b, cu, wo, wy = _inputs(world)
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta, x, w, b)]
    ref_o = gated_delta_rule(*leaves[:5], cu)
    ref_y = causal_conv1d_reference(leaves[5], leaves[6], leaves[7], cu, True)
    ((ref_o * wo).sum() + (ref_y * wy).sum()).backward()
    sl = slice(rank * T_LOCAL, (rank + 1) * T_LOCAL)
    loc = [t[sl].clone().requires_grad_() for t in (q, k, v, g, beta, x)]
    wl, bl = w.clone().requires_grad_(), b.clone().requires_grad_()
    o = gated_delta_rule_cp(*loc[:5], cu, dist.group.WORLD, chunk=16)
    y = causal_conv1d_cp(loc[5], wl, bl, cu, dist.group.WORLD, silu=True)
    valid = int(cu[-1])
    keep = max(0, min(T_LOCAL, valid - rank * T_LOCAL))              # outputs on padding are undefined
    torch.testing.assert_close(o[:keep], ref_o[sl][:keep], rtol=2e-3, atol=2e-4)
    torch.testing.assert_close(y[:keep], ref_y[sl][:keep], rtol=2e-3, atol=2e-4)
    mask = torch.zeros(T_LOCAL, 1, 1, dtype=torch.float64)
    mask[:keep] = 1
    # the reference loss also counted padding rows; remove them on both sides
    ((o * wo[sl] * mask).sum() + (y * wy[sl] * mask[:, :, 0]).sum()).backward()
    leaves2 = [t.clone().requires_grad_() for t in (q, k, v, g, beta, x, w, b)]
    full_mask = torch.zeros(q.shape[0], 1, 1, dtype=torch.float64)
    full_mask[:valid] = 1
    ro = gated_delta_rule(*leaves2[:5], cu)
    ry = causal_conv1d_reference(leaves2[5], leaves2[6], leaves2[7], cu, True)
    ((ro * wo * full_mask).sum() + (ry * wy * full_mask[:, :, 0]).sum()).backward()
    for got, want in zip(loc, leaves2[:6]):
        torch.testing.assert_close(got.grad[:keep], want.grad[sl][:keep], rtol=2e-3, atol=2e-4)
    for got, want in ((wl, leaves2[6]), (bl, leaves2[7])):
        gsum = got.grad.clone()
        dist.all_reduce(gsum)
        torch.testing.assert_close(gsum, want.grad, rtol=2e-3, atol=2e-4)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 3])
def test_cp_delta_rule_and_conv_match_single_process(world):
    from dist_utils import run_distributed
    run_distributed(__file__, world)




def _worker_docs():
    """Per-document sharding (every document cut into `world` pieces), including 2-token pieces."""
    import datetime
    import torch.distributed as dist
    from xorl_b200.models.gated_deltanet import gated_delta_rule
    from xorl_b200.ops.seqmix import causal_conv1d_reference
    from xorl_b200.parallel.linear_attn_cp import causal_conv1d_cp_docs, gated_delta_rule_cp_docs
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    pieces = [2, 20, 1, 37]                                           # piece length of each document
    lens = [p * world for p in pieces]
    T = sum(lens)
    gcu = [0]
    for l in lens:
        gcu.append(gcu[-1] + l)
    f = lambda *s: torch.randn(*s, dtype=torch.float64)
    q = torch.nn.functional.normalize(f(T, H, DK), dim=-1)
    k = torch.nn.functional.normalize(f(T, H, DK), dim=-1)
    v, g, beta = f(T, H, DV), -torch.rand(T, H, dtype=torch.float64), torch.rand(T, H, dtype=torch.float64)
    x, w, wo, wy = f(T, C), f(C, K), f(T, H, DV), f(T, C)
    sel = torch.cat([torch.arange(gcu[d] + rank * p, gcu[d] + (rank + 1) * p) for d, p in enumerate(pieces)])
    lcu = [0]
    for p in pieces:
        lcu.append(lcu[-1] + p)
    full = [t.clone().requires_grad_() for t in (q, k, v, g, beta, x, w)]
    ro = gated_delta_rule(*full[:5], torch.tensor(gcu))
    ry = causal_conv1d_reference(full[5], full[6], None, torch.tensor(gcu), True)
    ((ro * wo).sum() + (ry * wy).sum()).backward()
    loc = [t[sel].clone().requires_grad_() for t in (q, k, v, g, beta, x)]
    wl = w.clone().requires_grad_()
    o = gated_delta_rule_cp_docs(*loc[:5], torch.tensor(lcu, dtype=torch.int32), dist.group.WORLD, chunk=16)
    y = causal_conv1d_cp_docs(loc[5], wl, None, torch.tensor(lcu, dtype=torch.int32), dist.group.WORLD, silu=True)
    torch.testing.assert_close(o, ro[sel], rtol=2e-3, atol=2e-4)
    torch.testing.assert_close(y, ry[sel], rtol=2e-3, atol=2e-4)
    ((o * wo[sel]).sum() + (y * wy[sel]).sum()).backward()
    for got, want in zip(loc, full[:6]):
        torch.testing.assert_close(got.grad, want.grad[sel], rtol=2e-3, atol=2e-4)
    gw = wl.grad.clone()
    dist.all_reduce(gw)
    torch.testing.assert_close(gw, full[6].grad, rtol=2e-3, atol=2e-4)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 3])
def test_cp_per_document_sharding_matches_single_process(world):
    from dist_utils import run_distributed
    run_distributed(__file__, world, "docs")


def _worker_ssd():
    import datetime
    import torch.distributed as dist
    from xorl_b200.models.mamba2 import segment_ids, ssd_reference
    from xorl_b200.parallel.linear_attn_cp import ssd_cp_docs
    dist.init_process_group("gloo", timeout=datetime.timedelta(seconds=120))
    rank, world = dist.get_rank(), dist.get_world_size()
    torch.manual_seed(0)
    pieces = [2, 20, 1, 37]
    gcu = [0]
    for p in pieces:
        gcu.append(gcu[-1] + p * world)
    T, Hh, P, G, N = gcu[-1], 4, 6, 2, 5
    f = lambda *s: torch.randn(*s, dtype=torch.float64)
    x, dt = f(T, Hh, P), torch.rand(T, Hh, dtype=torch.float64) * 0.5 + 0.01
    A, Bm, Cm, Dv, wy = -torch.rand(Hh, dtype=torch.float64) - 0.1, f(T, G, N), f(T, G, N), f(Hh), f(T, Hh, P)
    sel = torch.cat([torch.arange(gcu[d] + rank * p, gcu[d] + (rank + 1) * p) for d, p in enumerate(pieces)])
    lcu = [0]
    for p in pieces:
        lcu.append(lcu[-1] + p)
    full = [t.clone().requires_grad_() for t in (x, dt, A, Bm, Cm, Dv)]
    ref = ssd_reference(*full, segment_ids(torch.tensor(gcu), T))
    (ref * wy).sum().backward()
    loc = [t[sel].clone().requires_grad_() for t in (x, dt)]
    Al, Dl = A.clone().requires_grad_(), Dv.clone().requires_grad_()
    Bl, Cl = Bm[sel].clone().requires_grad_(), Cm[sel].clone().requires_grad_()
    y = ssd_cp_docs(loc[0], loc[1], Al, Bl, Cl, Dl, torch.tensor(lcu, dtype=torch.int32), dist.group.WORLD, chunk=8)
    torch.testing.assert_close(y.double(), ref[sel].double(), rtol=2e-3, atol=2e-4)
    (y * wy[sel]).sum().backward()
    for got, want in ((loc[0], full[0]), (loc[1], full[1]), (Bl, full[3]), (Cl, full[4])):
        torch.testing.assert_close(got.grad.double(), want.grad[sel].double(), rtol=2e-3, atol=2e-4)
    for got, want in ((Al, full[2]), (Dl, full[5])):
        gsum = got.grad.clone()
        dist.all_reduce(gsum)
        torch.testing.assert_close(gsum.double(), want.grad.double(), rtol=2e-3, atol=2e-4)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.distributed
@pytest.mark.parametrize("world", [2, 3])
def test_cp_mamba2_scan_matches_single_process(world):
    from dist_utils import run_distributed
    run_distributed(__file__, world, "ssd")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "docs":
        _worker_docs()
    elif len(sys.argv) > 1 and sys.argv[1] == "ssd":
        _worker_ssd()
    else:
        _worker()
