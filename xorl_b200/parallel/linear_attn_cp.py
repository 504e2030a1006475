"""Context parallelism for the linear-attention mixers (GatedDeltaNet): contiguous sequence shards
whose recurrent state and convolution tails are handed from rank to rank.

Rank r of a group of R holds the global tokens [r * T, (r + 1) * T) of the packed batch.  A document
that straddles a shard border needs, on the later rank,

* the last K - 1 inputs of the previous rank for the short convolution (``conv_halo``), and
* the recurrent state S [H, dk, dv] at the border.

The state leaving a shard is an affine function of the state entering it, S_out = M S_in + B, with
M [H, dk, dk] and B [H, dk, dv] that depend only on the shard's own tokens (M = 0 as soon as a
document starts inside the shard).  Every rank evaluates its (M, B) in one pass of the chunked
delta rule over its last document with the value vectors widened by dk zero columns and the start
state [0 | I]; one all-gather of the pairs lets each rank fold the maps of the ranks before it, and
a second pass produces the outputs from the true entering state.  No rank waits for another rank's
scan: the exchange is one collective, not a chain of R sends.  Gradients flow back through the
all-gather (sum of the gathered gradients per source rank).

Same role as the reference's operator-level linear-attention CP
(src/xorl/ops/linear_attention/ops/cp/context.py:13-139 for the shard bookkeeping,
cp/chunk_delta_h.py:1064-1231 for the per-rank transfer pairs and their merge, cp/comm.py:147-151
for the convolution tails)."""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist


def shard_documents(global_cu: List[int], lo: int, hi: int) -> Tuple[List[int], bool]:
    """Document boundaries of the global packed batch clipped to tokens [lo, hi), in local
    coordinates (always starting with 0 and ending with hi - lo), and whether the first local
    document began before ``lo``."""
    cuts = [0]
    for c in global_cu:
        if lo < c < hi:
            cuts.append(c - lo)
    cuts.append(hi - lo)
    starts_here = any(c == lo for c in global_cu[:-1])
    beyond = lo >= global_cu[-1]                      # padding behind the last document
    return sorted(set(cuts)), (not starts_here) and not beyond and lo > 0


class _AllGather(torch.autograd.Function):
    """[...] -> [R, ...]; backward sums the gathered gradients and keeps this rank's slice."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        world = dist.get_world_size(group)
        out = [torch.empty_like(x) for _ in range(world)]
        dist.all_gather(out, x.contiguous(), group=group)
        return torch.stack(out, 0)

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g[dist.get_rank(ctx.group)], None


def all_gather_with_grad(x: torch.Tensor, group) -> torch.Tensor:
    return _AllGather.apply(x, group)


def conv_halo(x: torch.Tensor, taps: int, group) -> torch.Tensor:
    """The last ``taps - 1`` rows of the previous rank's ``x`` (zeros on rank 0).  Differentiable:
    the gradient of a halo row returns to the rank that owns the row."""
    n = taps - 1
    if n <= 0:
        return x.new_zeros((0, x.shape[1]))
    tails = all_gather_with_grad(x[-n:], group)                      # [R, n, C]
    r = dist.get_rank(group)
    # rank 0 keeps the gather in its graph too (times zero): every rank must enter the backward
    # collective
    return tails[r - 1] if r > 0 else tails[0] * 0.0


def shard_transfer(q, k, v, g, beta, local_cu: List[int], continues_prev: bool, chunk: int):
    """(M [H, dk, dk], B [H, dk, dv]) of this shard: state after its last token = M S_in + B."""
    from ..models.gated_deltanet import gated_delta_rule_chunked
    T, H, dk = q.shape
    dv = v.shape[-1]
    s = local_cu[-2]                                                   # start of the last document
    e = local_cu[-1]
    sl = slice(s, e)
    cu = torch.tensor([0, e - s], dtype=torch.int32)
    whole = (s == 0 and continues_prev)
    if not whole:
        _, B = gated_delta_rule_chunked(q[sl], k[sl], v[sl], g[sl], beta[sl], cu, chunk,
                                        return_final_state=True)
        return torch.zeros(H, dk, dk, dtype=torch.float32, device=q.device), B
    v_wide = torch.cat([v[sl].float(), torch.zeros(e - s, H, dk, device=q.device)], dim=-1)
    S0 = torch.cat([torch.zeros(H, dk, dv, device=q.device),
                    torch.eye(dk, device=q.device).expand(H, dk, dk)], dim=-1)
    _, S = gated_delta_rule_chunked(q[sl], k[sl], v_wide, g[sl], beta[sl], cu, chunk,
                                    initial_state=S0, return_final_state=True)
    return S[..., dv:], S[..., :dv]


def entering_state(M_all: torch.Tensor, B_all: torch.Tensor, rank: int) -> torch.Tensor:
    """Fold the maps of ranks 0 .. rank-1, starting from an empty state."""
    S = torch.zeros_like(B_all[0])
    for j in range(rank):
        S = M_all[j] @ S + B_all[j]
    return S


def gated_delta_rule_cp(q, k, v, g, beta, global_cu, group, chunk: int = 64,
                        rank: Optional[int] = None, world: Optional[int] = None):
    """Gated delta rule over this rank's contiguous shard of a packed batch.

    q, k [T, H, dk], v [T, H, dv], g, beta [T, H] are the local tokens (every rank holds the same
    T); ``global_cu`` are the document boundaries of the whole batch.  Returns o [T, H, dv]."""
    from ..models.gated_deltanet import gated_delta_rule_chunked
    rank = dist.get_rank(group) if rank is None else rank
    world = dist.get_world_size(group) if world is None else world
    T = q.shape[0]
    gcu = [int(c) for c in (global_cu.tolist() if torch.is_tensor(global_cu) else global_cu)]
    local_cu, continues_prev = shard_documents(gcu, rank * T, (rank + 1) * T)
    M, B = shard_transfer(q, k, v, g, beta, local_cu, continues_prev, chunk)
    dk = q.shape[-1]
    MB = all_gather_with_grad(torch.cat([M, B.float()], dim=-1), group)      # one collective
    M_all, B_all = MB[..., :dk], MB[..., dk:]
    # a rank that starts with a new document ignores the entering state but still takes part in
    # the backward collective (zero state, same graph)
    S_in = entering_state(M_all, B_all, rank) + 0.0 * MB.sum()
    if not continues_prev:
        S_in = S_in * 0.0
    cu = torch.tensor(local_cu, dtype=torch.int32)
    return gated_delta_rule_chunked(q, k, v, g, beta, cu, chunk, initial_state=S_in)


def causal_conv1d_cp(x, weight, bias, global_cu, group, silu: bool = True):
    """Short convolution over a contiguous shard: the previous rank's last K - 1 rows are put in
    front, documents are cut on the global boundaries, and the halo rows are dropped again."""
    from ..ops.seqmix import causal_conv1d
    rank, T = dist.get_rank(group), x.shape[0]
    n = weight.shape[1] - 1
    halo = conv_halo(x, weight.shape[1], group)
    gcu = [int(c) for c in (global_cu.tolist() if torch.is_tensor(global_cu) else global_cu)]
    lo = rank * T - n
    local_cu, _ = shard_documents([c for c in gcu], max(lo, 0), (rank + 1) * T)
    if lo < 0:                                                         # rank 0: the halo is padding
        local_cu = [0] + [c + n for c in local_cu]
        local_cu = sorted(set(local_cu))
    ext = torch.cat([halo, x], 0)
    y = causal_conv1d(ext, weight, bias, torch.tensor(local_cu, dtype=torch.int32, device=x.device), silu=silu)
    return y[n:]


# ---- per-document sharding (the trainer's Ulysses layout) ---------------------------------------
def gated_delta_rule_cp_docs(q, k, v, g, beta, local_cu, group, chunk: int = 64):
    """Every document of the packed batch is cut into R contiguous pieces and this rank holds piece
    ``rank`` of each; ``local_cu`` delimits the local pieces.  One widened pass gives the affine
    map (M, B) of every local piece, one all-gather exchanges them, each rank folds the maps of the
    earlier pieces per document and a second pass produces the outputs."""
    from ..models.gated_deltanet import gated_delta_rule_chunked
    rank = dist.get_rank(group)
    T, H, dk = q.shape
    dv = v.shape[-1]
    cu = local_cu.cpu() if torch.is_tensor(local_cu) else torch.tensor(local_cu)
    D = cu.numel() - 1
    v_wide = torch.cat([v.float(), torch.zeros(T, H, dk, device=q.device)], dim=-1)
    S0 = torch.cat([torch.zeros(H, dk, dv, device=q.device),
                    torch.eye(dk, device=q.device).expand(H, dk, dk)], dim=-1).expand(D, H, dk, dk + dv)
    _, S = gated_delta_rule_chunked(q, k, v_wide, g, beta, cu, chunk, initial_state=S0,
                                    return_final_state="all")                # [D, H, dk, dv + dk]
    MB = all_gather_with_grad(S, group)                                       # [R, D, H, dk, dv + dk]
    B_all, M_all = MB[..., :dv], MB[..., dv:]
    S_in = torch.zeros(D, H, dk, dv, dtype=torch.float32, device=q.device) + 0.0 * MB.sum()
    for j in range(rank):
        S_in = M_all[j] @ S_in + B_all[j]
    return gated_delta_rule_chunked(q, k, v, g, beta, cu, chunk, initial_state=S_in)


def causal_conv1d_cp_docs(x, weight, bias, local_cu, group, silu: bool = True):
    """Short convolution under the same per-document sharding: in front of every local piece go
    the last K - 1 tokens of the document's earlier pieces (from as many earlier ranks as needed
    when pieces are shorter than K - 1)."""
    from ..ops.seqmix import causal_conv1d
    rank = dist.get_rank(group)
    n = weight.shape[1] - 1
    cu = [int(c) for c in (local_cu.tolist() if torch.is_tensor(local_cu) else local_cu)]
    D, C = len(cu) - 1, x.shape[1]
    if n <= 0:
        return causal_conv1d(x, weight, bias, torch.tensor(cu, dtype=torch.int32, device=x.device), silu=silu)
    tails = []
    for s, e in zip(cu[:-1], cu[1:]):
        take = min(e - s, n)
        t = x[e - take:e]
        if take < n:
            t = torch.cat([x.new_zeros((n - take, C)), t], 0)
        tails.append(t)
    gathered = all_gather_with_grad(torch.stack(tails, 0), group)            # [R, D, n, C]
    parts, ext_cu, keep = [], [0], []
    for d, (s, e) in enumerate(zip(cu[:-1], cu[1:])):
        p = e - s
        rows, need, j = [], n, rank - 1
        while need > 0 and j >= 0 and p > 0:
            t = min(p, need)
            rows.insert(0, gathered[j, d, n - t:n])
            need -= t
            j -= 1
        if need > 0:
            rows.insert(0, gathered[rank, d, :need] * 0.0)                   # document start: zeros
        parts += rows + [x[s:e]]
        base = ext_cu[-1]
        keep.append(torch.arange(base + n, base + n + p))
        ext_cu.append(base + n + p)
    ext = torch.cat(parts, 0)
    y = causal_conv1d(ext, weight, bias, torch.tensor(ext_cu, dtype=torch.int32, device=x.device), silu=silu)
    return y[torch.cat(keep).to(x.device)]


def ssd_cp_docs(x, dt, A, B, C, D, local_cu, group, chunk: int = 128):
    """Mamba2 scan under per-document sharding.  The state update S_t = a_t S_{t-1} + dt_t x_t (x) B_t
    has a scalar decay per head, so a piece's map is (prod a, state reached from zero): the local
    scan runs from a zero state, the pieces' (log-decay, end state) pairs are all-gathered, every
    rank folds the earlier pieces of each document into the state entering its piece, and adds the
    missing term  y_t += (prod_{tau <= t} a_tau) * S_in C_t  to its outputs.

    x [T, H, P], dt [T, H] (after softplus / clamp), A [H], B, C [T, G, N], D [H] -> y [T, H, P] fp32."""
    from ..models.mamba2 import segment_ids, ssd_chunked
    rank = dist.get_rank(group)
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    cu = (local_cu.cpu() if torch.is_tensor(local_cu) else torch.tensor(local_cu)).to(torch.int64)
    n_docs = cu.numel() - 1
    seg = segment_ids(cu.to(x.device), T)
    y = ssd_chunked(x, dt, A, B, C, D, seg, chunk)
    la = dt.float() * A.float()                                             # log a_t  [T, H]
    cs = torch.cat([la.new_zeros(1, H), la.cumsum(0)], 0)                   # exclusive prefix sums
    cud = cu.to(x.device)
    base, end = cs[cud[:-1]], cs[cud[1:]]                                   # [D, H]
    inc = cs[1:] - base[seg]                                                # log decay from piece start through t
    total = end - base                                                      # log decay of the whole piece
    w = torch.exp(total[seg] - inc) * dt.float()                            # weight of token t in the end state
    xf, Bh, Ch = x.float(), B.float().repeat_interleave(rep, 1), C.float().repeat_interleave(rep, 1)
    bounds = list(zip(cu[:-1].tolist(), cu[1:].tolist()))
    ends = [torch.einsum("thp,thn->hpn", w[s:e].unsqueeze(-1) * xf[s:e], Bh[s:e]) for s, e in bounds]
    S_end = torch.stack(ends, 0) if ends else xf.new_zeros(0, H, P, N)
    packed = torch.cat([S_end.reshape(n_docs, H, P * N), total.unsqueeze(-1)], dim=-1)
    allp = all_gather_with_grad(packed, group)                              # [R, D, H, P*N + 1]
    S_in = torch.zeros(n_docs, H, P, N, dtype=torch.float32, device=x.device) + 0.0 * allp.sum()
    for j in range(rank):
        S_in = torch.exp(allp[j][..., -1]).view(n_docs, H, 1, 1) * S_in + allp[j][..., :-1].reshape(n_docs, H, P, N)
    parts = [torch.exp(inc[s:e]).unsqueeze(-1) * torch.einsum("hpn,thn->thp", S_in[d], Ch[s:e])
             for d, (s, e) in enumerate(bounds)]
    if parts:
        y = y + torch.cat(parts, 0)
    return y
