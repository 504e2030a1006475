"""Mamba2 (state-space duality) token mixer over packed sequences.

Per head h with state ``S [P, N]`` (P = head dim, N = state size), inside each document:

    S_t = exp(dt_t * A_h) * S_{t-1} + dt_t * x_t (outer) B_t
    y_t = S_t C_t + D_h * x_t

``B`` and ``C`` are shared by the heads of a group.  ``ssd_chunked`` evaluates the recurrence in
chunks of Q tokens: a masked quadratic form inside each chunk (GEMM-shaped) plus one state per chunk
carried across chunk borders; documents are kept apart by comparing segment ids instead of by
infinite decays, so packed batches need no special values.  ``ssd_reference`` is the token-by-token
recurrence the chunked form is tested against.

The layer follows the layout of the reference's mixer (src/xorl/ops/ssm/layers/mamba2_mixer.py):
one input projection producing ``[gate | x | B | C | dt]``, a causal depthwise convolution + SiLU
over ``[x | B | C]``, ``dt = clamp(softplus(dt + dt_bias))``, the scan, a gated grouped RMSNorm
(``weight * group_rmsnorm(y * silu(gate))``, src/xorl/ops/ssm/modules/gated_norm.py) and the output
projection.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from .config import ModelConfig
from .context import StepContext
from ..ops.seqmix import causal_conv1d
from .layers import Linear


def segment_ids(cu_seqlens: torch.Tensor, T: int) -> torch.Tensor:
    """Document index of every token; tokens past the last boundary form their own segment."""
    pos = torch.arange(T, device=cu_seqlens.device)
    return torch.searchsorted(cu_seqlens.to(torch.int64).contiguous(), pos, right=True) - 1


def ssd_reference(x, dt, A, B, C, D, seg) -> torch.Tensor:
    """x [T,H,P], dt [T,H], A [H], B/C [T,G,N], D [H], seg [T] -> y [T,H,P] (fp32)."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    x, dt, B, C = x.float(), dt.float(), B.float(), C.float()
    S = torch.zeros(H, P, N, dtype=torch.float32, device=x.device)
    out = []
    for t in range(T):
        if t > 0 and seg[t] != seg[t - 1]:
            S = torch.zeros_like(S)
        Bt = B[t].repeat_interleave(rep, 0)                     # [H, N]
        Ct = C[t].repeat_interleave(rep, 0)
        S = S * torch.exp(dt[t] * A.float()).view(H, 1, 1) + (dt[t].view(H, 1) * x[t]).unsqueeze(-1) * Bt.unsqueeze(1)
        out.append((S * Ct.unsqueeze(1)).sum(-1) + D.float().view(H, 1) * x[t])
    return torch.stack(out, 0)


def ssd_chunked(x, dt, A, B, C, D, seg, chunk: int = 128) -> torch.Tensor:
    """Same contract as ``ssd_reference``, O(T * chunk) work in GEMM-shaped pieces."""
    T, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    rep = H // G
    Q = chunk
    pad = (-T) % Q
    x32, dt32, B32, C32 = x.float(), dt.float(), B.float(), C.float()
    if pad:
        x32 = F.pad(x32, (0, 0, 0, 0, 0, pad))
        dt32 = F.pad(dt32, (0, 0, 0, pad))
        B32 = F.pad(B32, (0, 0, 0, 0, 0, pad))
        C32 = F.pad(C32, (0, 0, 0, 0, 0, pad))
        seg = torch.cat([seg, seg.new_full((pad,), int(seg[-1]) + 1)])
    nc = (T + pad) // Q
    xc = x32.view(nc, Q, H, P)
    dtc = dt32.view(nc, Q, H)
    Bc = B32.view(nc, Q, G, N)
    Cc = C32.view(nc, Q, G, N)
    sg = seg.view(nc, Q)
    a = dtc * A.float().view(1, 1, H)                            # log decay per token  [nc,Q,H]
    cs = torch.cumsum(a, dim=1)                                  # inclusive
    # ---- inside a chunk: y_i += sum_{j<=i, same doc} exp(cs_i - cs_j) (C_i . B_j) dt_j x_j
    same = sg.unsqueeze(2) == sg.unsqueeze(1)                    # [nc,Q,Q]
    causal = torch.ones(Q, Q, dtype=torch.bool, device=x.device).tril()
    mask = (same & causal).unsqueeze(-1)                         # [nc,Q,Q,1]
    diff = cs.unsqueeze(2) - cs.unsqueeze(1)                     # [nc,Q(i),Q(j),H]
    L = torch.exp(diff.masked_fill(~mask, float("-inf")))        # masked entries become exactly 0
    cb = torch.einsum("cign,cjgn->cijg", Cc, Bc).repeat_interleave(rep, dim=3)     # [nc,Q,Q,H]
    xdt = xc * dtc.unsqueeze(-1)                                 # [nc,Q,H,P]
    y = torch.einsum("cijh,cjhp->cihp", L * cb, xdt)
    # ---- state contributed by each chunk at its end (tokens of the chunk's last document only)
    end_seg = sg[:, -1]                                          # [nc]
    to_end = torch.exp((cs[:, -1:, :] - cs).masked_fill((sg != end_seg.unsqueeze(1)).unsqueeze(-1), float("-inf")))
    Bh = Bc.repeat_interleave(rep, dim=2)                        # [nc,Q,H,N]
    Ch = Cc.repeat_interleave(rep, dim=2)
    S_chunk = torch.einsum("cjh,cjhp,cjhn->chpn", to_end, xdt, Bh)                 # [nc,H,P,N]
    # ---- carry the state across chunks; it survives a chunk only if no document starts in it
    chunk_decay = torch.exp(cs[:, -1, :])                        # [nc,H]
    prev_end = torch.cat([sg.new_full((1,), -1), end_seg[:-1]])  # segment of the token before the chunk
    carry_in = []
    R = torch.zeros(H, P, N, dtype=torch.float32, device=x.device)
    for c in range(nc):
        carry_in.append(R)
        keep = (end_seg[c] == prev_end[c]).to(torch.float32)
        R = R * (chunk_decay[c].view(H, 1, 1) * keep) + S_chunk[c]
    Rin = torch.stack(carry_in, 0)                               # [nc,H,P,N]
    from_start = torch.exp(cs.masked_fill((sg != prev_end.unsqueeze(1)).unsqueeze(-1), float("-inf")))  # [nc,Q,H]
    y = y + torch.einsum("cih,cihn,chpn->cihp", from_start, Ch, Rin)
    y = y + D.float().view(1, 1, H, 1) * xc
    return y.reshape(nc * Q, H, P)[:T]


def gated_group_rmsnorm(y: torch.Tensor, gate: torch.Tensor, weight: torch.Tensor, group_size: int,
                        eps: float) -> torch.Tensor:
    """weight * rmsnorm_per_group(y * silu(gate)), statistics in fp32."""
    h = y.float() * F.silu(gate.float())
    shp = h.shape
    h = h.view(*shp[:-1], shp[-1] // group_size, group_size)
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    return weight * h.view(shp).to(y.dtype)


class Mamba2Mixer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        x = cfg.extra
        self.H, self.P = x["mamba_num_heads"], x["mamba_head_dim"]
        self.G, self.N = x.get("n_groups", 1), x["ssm_state_size"]
        self.K = x.get("conv_kernel", 4)
        self.chunk = x.get("chunk_size", 128)
        lim = x.get("time_step_limit") or (0.0, float("inf"))
        self.dt_limit = (float(lim[0]), float(lim[1]))
        self.eps = cfg.rms_norm_eps
        if self.H % self.G:
            raise ValueError(f"n_groups={self.G} must divide mamba_num_heads={self.H}")
        self.d_inner = self.H * self.P
        self.conv_dim = self.d_inner + 2 * self.G * self.N
        bias = bool(x.get("use_bias", False))
        self.in_proj = Linear(cfg.hidden_size, self.d_inner + self.conv_dim + self.H, bias=bias, dtype=dtype, device=device)
        self.conv1d_weight = nn.Parameter(torch.empty(self.conv_dim, self.K, dtype=dtype, device=device))
        self.conv1d_bias = nn.Parameter(torch.zeros(self.conv_dim, dtype=dtype, device=device)) \
            if x.get("use_conv_bias", True) else None
        self.dt_bias = nn.Parameter(torch.ones(self.H, dtype=dtype, device=device))
        self.A_log = nn.Parameter(torch.zeros(self.H, dtype=dtype, device=device))
        self.D = nn.Parameter(torch.ones(self.H, dtype=dtype, device=device))
        self.norm_weight = nn.Parameter(torch.ones(self.d_inner, dtype=dtype, device=device))
        self.out_proj = Linear(self.d_inner, cfg.hidden_size, bias=bias, dtype=dtype, device=device)
        for p in (self.dt_bias, self.A_log, self.D, self.norm_weight):
            p._xb_no_decay = True

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T = h.shape[0]
        cp_group = None
        if ctx.cp is not None:
            # Ulysses sharding (rank u holds piece u of every document): convolution tails and scan
            # states cross the ranks per document (parallel/linear_attn_cp.py)
            if getattr(ctx.cp, "R", 1) > 1:
                raise NotImplementedError("Mamba2 layers do not run under ring (zigzag) context parallelism: "
                                          "use ulysses_parallel_size instead")
            cp_group = ctx.cp.u_group
            local_cu = ctx.aux["local_cu_seqlens"]
        proj = self.in_proj(h)
        gate, xbc, dt = proj.split([self.d_inner, self.conv_dim, self.H], dim=-1)
        if cp_group is not None:
            from ..parallel.linear_attn_cp import causal_conv1d_cp_docs, ssd_cp_docs
            xbc = causal_conv1d_cp_docs(xbc.contiguous(), self.conv1d_weight, self.conv1d_bias, local_cu,
                                        cp_group, silu=True)
        else:
            xbc = causal_conv1d(xbc.contiguous(), self.conv1d_weight, self.conv1d_bias, ctx.cu_seqlens, silu=True)
        x, B, C = xbc.split([self.d_inner, self.G * self.N, self.G * self.N], dim=-1)
        dt = torch.clamp(F.softplus(dt.float() + self.dt_bias.float()), self.dt_limit[0], self.dt_limit[1])
        A = -torch.exp(self.A_log.float())
        if cp_group is not None:
            y = ssd_cp_docs(x.reshape(T, self.H, self.P), dt, A, B.reshape(T, self.G, self.N),
                            C.reshape(T, self.G, self.N), self.D, local_cu, cp_group, self.chunk)
        else:
            seg = segment_ids(ctx.cu_seqlens, T)
            y = ssd_chunked(x.reshape(T, self.H, self.P), dt, A, B.reshape(T, self.G, self.N),
                            C.reshape(T, self.G, self.N), self.D, seg, self.chunk)
        y = gated_group_rmsnorm(y.reshape(T, self.d_inner).to(h.dtype), gate, self.norm_weight,
                                self.d_inner // self.G, self.eps)
        return self.out_proj(y.to(h.dtype))


def init_mamba_parameter_(name: str, p: torch.Tensor, gen: torch.Generator, time_step_min=1e-3,
                          time_step_max=0.1, time_step_floor=1e-4) -> bool:
    """Initial values of the state-space parameters (src/xorl/models/transformers/nemotron_h/
    modeling_nemotron_h.py, ``_init_weights``): A = 1..H, D = 1, dt_bias = softplus^-1 of a
    log-uniform step size.  Returns False for names it does not own."""
    leaf = name.rsplit(".", 1)[-1]
    if leaf == "A_log":
        p.copy_(torch.log(torch.arange(1, p.numel() + 1, dtype=torch.float32)).to(p.dtype))
    elif leaf == "D" or leaf == "norm_weight":
        p.fill_(1.0)
    elif leaf == "dt_bias":
        u = torch.rand(p.numel(), generator=gen)
        dt = torch.exp(u * (math.log(time_step_max) - math.log(time_step_min)) + math.log(time_step_min))
        dt = dt.clamp(min=time_step_floor)
        p.copy_((dt + torch.log(-torch.expm1(-dt))).to(p.dtype))
    elif leaf == "conv1d_bias":
        p.zero_()
    else:
        return False
    return True
