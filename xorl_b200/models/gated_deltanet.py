"""Gated DeltaNet token mixer (Qwen3-Next / Qwen3.5 "linear_attention" layers).

Per head a matrix state S [d_k, d_v] follows the gated delta rule

    S_t = exp(g_t) * S_{t-1} + k_t (x) [ beta_t * (v_t - (exp(g_t) * S_{t-1})^T k_t) ],      o_t = S_t^T q_t

with q, k passed through a causal depthwise convolution + SiLU, L2-normalised (q also scaled by
d_k^-1/2), beta = sigmoid(b x), g = -exp(A_log) * softplus(a x + dt_bias), and the output
RMS-normalised per head and gated by SiLU(z) before the output projection
(src/xorl/ops/linear_attention/layers/gated_deltanet.py:46-470).

This is a plain PyTorch implementation: the recurrence runs token by token inside every document of
the packed batch (state reset at document boundaries, convolution not crossing them), vectorised
over heads.  It is exact and differentiable, and meant for functional coverage and small-scale
runs; the reference's chunked Triton kernels have no CUDA counterpart here yet."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from .config import ModelConfig
from .context import StepContext
from .layers import Linear


def causal_depthwise_conv(x: torch.Tensor, weight: torch.Tensor, cu_seqlens) -> torch.Tensor:
    """x [T, C], weight [C, K]: y[t, c] = sum_j w[c, j] * x[t - (K-1) + j, c] inside each document."""
    K = weight.shape[1]
    out = torch.empty_like(x)
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        if e <= s:
            continue
        xb = F.pad(x[s:e].t().unsqueeze(0), (K - 1, 0))                  # [1, C, L + K - 1]
        out[s:e] = F.conv1d(xb, weight.unsqueeze(1).to(x.dtype), groups=x.shape[1])[0].t()
    return out


def gated_delta_rule(q, k, v, g, beta, cu_seqlens):
    """q, k [T, H, dk], v [T, H, dv], g, beta [T, H] -> o [T, H, dv].  fp32 state."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    out = []
    cu = cu_seqlens.tolist()
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device)
        for t in range(s, e):
            S = S * torch.exp(g[t].float()).view(H, 1, 1)
            kt, vt = k[t].float(), v[t].float()
            pred = torch.einsum("hkv,hk->hv", S, kt)
            delta = (vt - pred) * beta[t].float().unsqueeze(-1)
            S = S + kt.unsqueeze(-1) * delta.unsqueeze(1)
            out.append(torch.einsum("hkv,hk->hv", S, q[t].float()))
    if cu[-1] < T:                                                         # tokens outside every document
        out += [torch.zeros(H, dv, device=q.device)] * (T - cu[-1])
    return torch.stack(out, 0).to(v.dtype)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        x = cfg.extra
        self.layer_idx = layer_idx
        self.Hk, self.Hv = x["linear_num_key_heads"], x["linear_num_value_heads"]
        self.dk, self.dv = x["linear_key_head_dim"], x["linear_value_head_dim"]
        self.K = x.get("linear_conv_kernel_dim", 4)
        self.key_dim, self.value_dim = self.Hk * self.dk, self.Hv * self.dv
        H = cfg.hidden_size
        kw = dict(dtype=dtype, device=device)
        self.q_proj = Linear(H, self.key_dim, **kw)
        self.k_proj = Linear(H, self.key_dim, **kw)
        self.v_proj = Linear(H, self.value_dim, **kw)
        self.a_proj = Linear(H, self.Hv, **kw)
        self.b_proj = Linear(H, self.Hv, **kw)
        self.g_proj = Linear(H, self.value_dim, **kw)
        self.q_conv1d = nn.Parameter(torch.empty(self.key_dim, self.K, **kw))
        self.k_conv1d = nn.Parameter(torch.empty(self.key_dim, self.K, **kw))
        self.v_conv1d = nn.Parameter(torch.empty(self.value_dim, self.K, **kw))
        self.A_log = nn.Parameter(torch.empty(self.Hv, dtype=torch.float32, device=device))
        self.dt_bias = nn.Parameter(torch.empty(self.Hv, dtype=torch.float32, device=device))
        self.o_norm_weight = nn.Parameter(torch.ones(self.dv, **kw))
        self.o_proj = Linear(self.value_dim, H, **kw)
        self.eps = cfg.rms_norm_eps

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T = x.shape[0]
        cu = ctx.cu_seqlens
        q = F.silu(causal_depthwise_conv(self.q_proj(x), self.q_conv1d, cu))
        k = F.silu(causal_depthwise_conv(self.k_proj(x), self.k_conv1d, cu))
        v = F.silu(causal_depthwise_conv(self.v_proj(x), self.v_conv1d, cu))
        beta = torch.sigmoid(self.b_proj(x).float())
        g = -torch.exp(self.A_log.float()) * F.softplus(self.a_proj(x).float() + self.dt_bias.float())
        q = F.normalize(q.view(T, self.Hk, self.dk).float(), dim=-1) * self.dk ** -0.5
        k = F.normalize(k.view(T, self.Hk, self.dk).float(), dim=-1)
        if self.Hv > self.Hk:
            rep = self.Hv // self.Hk
            q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
        o = gated_delta_rule(q, k, v.view(T, self.Hv, self.dv), g, beta, cu).float()
        z = self.g_proj(x).view(T, self.Hv, self.dv).float()
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps) * self.o_norm_weight.float()
        o = (o * F.silu(z)).to(x.dtype)
        return self.o_proj(o.reshape(T, self.value_dim))
