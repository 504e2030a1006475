"""Gated DeltaNet token mixer (Qwen3-Next / Qwen3.5 "linear_attention" layers).

Per head a matrix state S [d_k, d_v] follows the gated delta rule

    S_t = exp(g_t) * S_{t-1} + k_t (x) [ beta_t * (v_t - (exp(g_t) * S_{t-1})^T k_t) ],      o_t = S_t^T q_t

with q, k passed through a causal depthwise convolution + SiLU, L2-normalised (q also scaled by
d_k^-1/2), beta = sigmoid(b x), g = -exp(A_log) * softplus(a x + dt_bias), and the output
RMS-normalised per head and gated by SiLU(z) before the output projection
(src/xorl/ops/linear_attention/layers/gated_deltanet.py:46-470).

``gated_delta_rule`` is the token-by-token recurrence (the definition, used as the test oracle).
``gated_delta_rule_chunked`` evaluates the same recurrence in chunks of 64 tokens: inside a chunk
the deltas u_t = beta_t (v_t - (exp(g_t) S_{t-1})^T k_t) solve a unit lower-triangular system
(I + diag(beta) A) U = diag(beta) (V - diag(gamma) K S_0), A[i, j] = gamma_i / gamma_j k_i.k_j for
j < i and gamma the running decay product, so every chunk costs a handful of batched matrix
products and only one [d_k, d_v] state per head crosses chunk borders (the chunked formulation of
src/xorl/ops/linear_attention/ops/gated_delta_rule/chunk.py).  Documents of the packed batch are cut
into chunks separately, so neither the state nor the convolution crosses a document start.  The
short convolutions run on the CUDA kernel of ``ops/seqmix.py`` when the activations are bf16 on a
GPU."""
from __future__ import annotations

import torch
import torch.nn.functional as F
from torch import nn

from ..ops.seqmix import causal_conv1d
from .config import ModelConfig
from .context import StepContext
from .layers import Linear

CHUNK = 64


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


def _chunk_index(cu, T: int, chunk: int, device):
    """Rows of token indices, one row per chunk of one document (``-1`` pads), and a flag per row
    that is 1 where the row opens a document."""
    rows, first, doc = [], [], []
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        for c0 in range(s, e, chunk):
            c1 = min(e, c0 + chunk)
            rows.append(list(range(c0, c1)) + [-1] * (chunk - (c1 - c0)))
            first.append(1.0 if c0 == s else 0.0)
            doc.append(b)
    if not rows:
        rows, first, doc = [[-1] * chunk], [1.0], [0]
    return (torch.tensor(rows, dtype=torch.long, device=device),
            torch.tensor(first, dtype=torch.float32, device=device), doc)


def gated_delta_rule_chunked(q, k, v, g, beta, cu_seqlens, chunk: int = CHUNK, initial_state=None,
                             return_final_state: bool = False):
    """Same contract as ``gated_delta_rule``.  ``initial_state`` [H, dk, dv] seeds the first
    document, or [D, H, dk, dv] seeds every document; with ``return_final_state`` the state after
    the last document's last token is returned as well, with ``return_final_state="all"`` the
    states after every document [D, H, dk, dv] (zeros for empty documents).  These are what
    context-parallel ranks exchange with their neighbours."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    cu = cu_seqlens.tolist()
    idx, first, doc_of = _chunk_index(cu, T, chunk, q.device)
    n_docs = len(cu) - 1
    per_doc = initial_state is not None and initial_state.dim() == 4
    N = idx.shape[0]
    valid = (idx >= 0)
    gi = idx.clamp_min(0)
    vm = valid.view(N, chunk, 1, 1).float()

    def take(x):                                           # [T, H, d] -> [N, H, C, d], pads zeroed
        return (x.float()[gi] * vm).permute(0, 2, 1, 3)

    Q, K, V = take(q), take(k), take(v)
    gg = (g.float()[gi] * vm[..., 0]).permute(0, 2, 1)                     # [N, H, C]
    bb = (beta.float()[gi] * vm[..., 0]).permute(0, 2, 1)
    G = gg.cumsum(-1)                                                       # log gamma
    tri = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    diff = (G.unsqueeze(-1) - G.unsqueeze(-2)).masked_fill(~tri, 0.0)
    decay = torch.exp(diff) * tri                                           # gamma_i / gamma_j, j <= i
    gamma = torch.exp(G)                                                    # [N, H, C]
    KK = K @ K.transpose(-1, -2)
    strict = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril(-1)
    L = bb.unsqueeze(-1) * (decay * KK) * strict                            # diag(beta) A
    eye = torch.eye(chunk, device=q.device)
    rhs = torch.cat([bb.unsqueeze(-1) * V, bb.unsqueeze(-1) * gamma.unsqueeze(-1) * K], dim=-1)
    sol = torch.linalg.solve_triangular(eye + L, rhs, upper=False, unitriangular=True)
    TV, W = sol[..., :dv], sol[..., dv:]                                    # [N,H,C,dv], [N,H,C,dk]
    Aqk = decay * (Q @ K.transpose(-1, -2))                                 # [N,H,C,C]
    Qg = gamma.unsqueeze(-1) * Q
    g_end = gamma[..., -1]                                                  # [N, H]
    Kdec = torch.exp(G[..., -1:] - G).unsqueeze(-1) * K                     # gamma_C / gamma_j k_j

    S = torch.zeros(H, dk, dv, dtype=torch.float32, device=q.device)
    zero_state = S
    outs = []
    finals = {}
    first_l = first.tolist()
    for n in range(N):
        if first_l[n] > 0:
            if per_doc:
                S = initial_state[doc_of[n]].float()
            elif n == 0 and initial_state is not None:
                S = initial_state.float()
            else:
                S = zero_state
        U = TV[n] - W[n] @ S
        outs.append(Qg[n] @ S + Aqk[n] @ U)
        S = g_end[n].view(H, 1, 1) * S + Kdec[n].transpose(-1, -2) @ U
        finals[doc_of[n]] = S
    O = torch.stack(outs, 0).permute(0, 2, 1, 3)                            # [N, C, H, dv]
    out = torch.zeros(T, H, dv, dtype=torch.float32, device=q.device)
    out = out.index_put((idx[valid],), O[valid])
    out = out.to(v.dtype)
    if return_final_state == "all":
        # a document without tokens leaves its entering state untouched
        return out, torch.stack([finals.get(d, initial_state[d].float() if per_doc else zero_state)
                                 for d in range(max(n_docs, 1))], 0)
    return (out, S) if return_final_state else out


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
        cp_group = None
        if ctx.cp is not None:
            # Ulysses sharding: every document is cut into contiguous pieces, rank u holds piece u;
            # states and convolution tails are handed over per document (parallel/linear_attn_cp.py)
            if getattr(ctx.cp, "R", 1) > 1:
                raise NotImplementedError("GatedDeltaNet layers do not run under ring (zigzag) context "
                                          "parallelism: use ulysses_parallel_size instead")
            from ..parallel.linear_attn_cp import causal_conv1d_cp_docs, gated_delta_rule_cp_docs
            cp_group = ctx.cp.u_group
            cu = ctx.aux["local_cu_seqlens"]
            conv = lambda t, w: causal_conv1d_cp_docs(t, w, None, cu, cp_group, silu=True)
        else:
            conv = lambda t, w: causal_conv1d(t, w, None, cu, silu=True)
        q = conv(self.q_proj(x), self.q_conv1d)
        k = conv(self.k_proj(x), self.k_conv1d)
        v = conv(self.v_proj(x), self.v_conv1d)
        beta = torch.sigmoid(self.b_proj(x).float())
        g = -torch.exp(self.A_log.float()) * F.softplus(self.a_proj(x).float() + self.dt_bias.float())
        q = F.normalize(q.view(T, self.Hk, self.dk).float(), dim=-1) * self.dk ** -0.5
        k = F.normalize(k.view(T, self.Hk, self.dk).float(), dim=-1)
        if self.Hv > self.Hk:
            rep = self.Hv // self.Hk
            q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)
        if cp_group is not None:
            o = gated_delta_rule_cp_docs(q, k, v.view(T, self.Hv, self.dv), g, beta, cu, cp_group).float()
        else:
            o = gated_delta_rule_chunked(q, k, v.view(T, self.Hv, self.dv), g, beta, cu).float()
        z = self.g_proj(x).view(T, self.Hv, self.dv).float()
        o = o * torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + self.eps) * self.o_norm_weight.float()
        o = (o * F.silu(z)).to(x.dtype)
        return self.o_proj(o.reshape(T, self.value_dim))
