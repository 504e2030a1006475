"""DeepSeek-V4: hyper-connected residual streams, shared-KV sparse attention over a sliding window
plus compressed keys, and a sqrt-softplus routed MoE with hash-routed first layers
(src/xorl/models/transformers/deepseek_v4/modeling_deepseek_v4.py, src/xorl/ops/dsv4/*).

Hyper-connections.  The residual stream holds ``hc_mult`` copies ``x [T, hc, H]``.  Before a
sub-layer three mixers are read off the stream itself (``mix = (x_flat @ fn^T) * rsqrt(mean x_flat^2)``,
no gradient): ``pre [hc]`` (sigmoid) collapses the copies into the sub-layer input, ``post [hc]``
(2 * sigmoid) spreads the sub-layer output back and ``comb [hc, hc]`` (softmax rows, then Sinkhorn
normalisation) mixes the copies among themselves: ``x'_i = post_i * y + sum_j comb[j, i] * x_j``.

Attention.  One key/value vector per token shared by all heads (K = V = ``kv_norm(wkv(x))``,
rotary embedding on the last ``qk_rope_head_dim`` channels), queries through a low-rank bottleneck
with a weight-free per-head RMS norm, one sink logit per head in the softmax denominator.  Every
query sees the last ``sliding_window`` tokens; layers with ``compress_ratio`` r also see compressed
entries: each group of r tokens is pooled by a learned softmax gate into one key (groups of ratio 4
overlap with the previous group), and for ratio 4 an indexer keeps the ``index_topk`` best groups
per query.  The rotary part of the output is rotated back by the query position, heads are projected
group-wise to ``o_lora_rank`` and then to the model width.

Everything here is plain PyTorch per document (masked softmax over window + compressed keys): the
functional definition of the family, not a tuned kernel.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F
from torch import nn

from ..ops import attention as attn_ops
from ..ops import moe as moe_ops
from .config import ModelConfig
from .context import StepContext
from .layers import MLP, Linear, RMSNorm
from .moe import MoEBlock


# ------------------------------------------------------------------------------------------------
# hyper-connections
# ------------------------------------------------------------------------------------------------
def hc_mixes(x: torch.Tensor, fn: torch.Tensor, eps: float) -> torch.Tensor:
    """x [T, hc, H] -> mixer logits [T, (2 + hc) * hc] (fp32)."""
    flat = x.flatten(1).float()
    return F.linear(flat, fn.float()) * torch.rsqrt(flat.square().mean(-1, keepdim=True) + eps)


def hc_split_sinkhorn(mixes, scale, base, hc: int, iters: int, eps: float):
    """(pre [T, hc], post [T, hc], comb [T, hc, hc]) from the mixer logits."""
    pre = torch.sigmoid(mixes[:, :hc] * scale[0] + base[:hc]) + eps
    post = 2.0 * torch.sigmoid(mixes[:, hc:2 * hc] * scale[1] + base[hc:2 * hc])
    comb = mixes[:, 2 * hc:2 * hc + hc * hc].reshape(-1, hc, hc) * scale[2] + base[2 * hc:].reshape(hc, hc)
    comb = torch.softmax(comb, dim=-1) + eps
    comb = comb / (comb.sum(-2, keepdim=True) + eps)
    for _ in range(iters - 1):
        comb = comb / (comb.sum(-1, keepdim=True) + eps)
        comb = comb / (comb.sum(-2, keepdim=True) + eps)
    return pre, post, comb


class HyperConnection(nn.Module):
    """Mixer parameters of one sub-layer (kept in fp32; they receive no gradient)."""

    def __init__(self, cfg: ModelConfig, device=None, head: bool = False):
        super().__init__()
        self.hc = int(cfg.extra.get("hc_mult", 4))
        self.iters = int(cfg.extra.get("hc_sinkhorn_iters", 20))
        self.hc_eps = float(cfg.extra.get("hc_eps", 1e-6))
        self.eps = cfg.rms_norm_eps
        self.head = head
        n = self.hc if head else (2 + self.hc) * self.hc
        self.fn = nn.Parameter(torch.zeros(n, self.hc * cfg.hidden_size, dtype=torch.float32, device=device),
                               requires_grad=False)
        self.base = nn.Parameter(torch.zeros(n, dtype=torch.float32, device=device), requires_grad=False)
        self.scale = nn.Parameter(torch.ones(1 if head else 3, dtype=torch.float32, device=device),
                                  requires_grad=False)

    @torch.no_grad()
    def mixers(self, x):
        m = hc_mixes(x, self.fn, self.eps)
        if self.head:
            return torch.sigmoid(m * self.scale[0] + self.base) + self.hc_eps
        return hc_split_sinkhorn(m, self.scale, self.base, self.hc, self.iters, self.hc_eps)

    def pre(self, x):
        """x [T, hc, H] -> (sub-layer input [T, H], post, comb)."""
        pre, post, comb = self.mixers(x)
        return (pre.unsqueeze(-1) * x.float()).sum(1).to(x.dtype), post, comb

    @staticmethod
    def post(y, x, post, comb):
        """y [T, H] sub-layer output, x [T, hc, H] stream before the sub-layer."""
        out = post.unsqueeze(-1) * y.float().unsqueeze(1) + torch.einsum("tji,tjh->tih", comb, x.float())
        return out.to(x.dtype)

    def collapse(self, x):
        return (self.mixers(x).unsqueeze(-1) * x.float()).sum(1).to(x.dtype)


# ------------------------------------------------------------------------------------------------
# rotary helpers (tables built from positions; pairs are interleaved in the checkpoint layout)
# ------------------------------------------------------------------------------------------------
def rope_tables(positions: torch.Tensor, dim: int, theta: float):
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, device=positions.device, dtype=torch.float32) / dim))
    ang = positions.float().unsqueeze(-1) * inv
    return ang.cos(), ang.sin()


def rope_tail(t: torch.Tensor, cos, sin, rd: int, inverse: bool = False) -> torch.Tensor:
    """Rotate the last ``rd`` channels of t [T, h, D] (interleaved pairs)."""
    T, h, D = t.shape
    tail = t[..., D - rd:].reshape(T, h, rd // 2, 2).transpose(-1, -2).reshape(T, h, rd)
    tail = attn_ops.rope_reference(tail, cos, -sin if inverse else sin)
    tail = tail.reshape(T, h, 2, rd // 2).transpose(-1, -2).reshape(T, h, rd)
    return torch.cat([t[..., :D - rd], tail], -1)


# ------------------------------------------------------------------------------------------------
# key compression and the indexer
# ------------------------------------------------------------------------------------------------
class Compressor(nn.Module):
    """Pools every ``ratio`` tokens into one vector with a learned softmax gate (+ a per-slot bias);
    with ratio 4 each group also sees the previous group through a second half of channels."""

    def __init__(self, cfg: ModelConfig, head_dim: int, ratio: int, dtype=None, device=None):
        super().__init__()
        self.ratio, self.hd = ratio, head_dim
        self.overlap = ratio == 4
        c = 2 if self.overlap else 1
        self.rd = cfg.extra["qk_rope_head_dim"]
        self.theta = float(cfg.extra.get("compress_rope_theta", cfg.rope_theta))
        self.eps = cfg.rms_norm_eps
        self.ape = nn.Parameter(torch.zeros(ratio, c * head_dim, dtype=dtype, device=device))
        self.wkv = Linear(cfg.hidden_size, c * head_dim, dtype=dtype, device=device)
        self.wgate = Linear(cfg.hidden_size, c * head_dim, dtype=dtype, device=device)
        self.norm = RMSNorm(head_dim, cfg.rms_norm_eps, dtype=dtype, device=device)

    def forward(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """One document x [L, H], positions [L] -> [L // ratio, head_dim] (may be empty)."""
        r, hd = self.ratio, self.hd
        G = x.shape[0] // r
        if G == 0:
            return x.new_zeros(0, hd)
        xf = x[:G * r].float()
        kv = F.linear(xf, self.wkv.weight.float()).view(G, r, -1)
        score = F.linear(xf, self.wgate.weight.float()).view(G, r, -1) + self.ape.float()
        if self.overlap:
            # slots 0..r-1: previous group (first half of channels); slots r..2r-1: this group (second half)
            kv2 = kv.new_zeros(G, 2 * r, hd)
            sc2 = score.new_full((G, 2 * r, hd), float("-inf"))
            kv2[:, r:], sc2[:, r:] = kv[..., hd:], score[..., hd:]
            kv2[1:, :r], sc2[1:, :r] = kv[:-1, :, :hd], score[:-1, :, :hd]
            kv, score = kv2, sc2
        pooled = (kv * score.softmax(1)).sum(1).to(x.dtype)
        pooled = self.norm(pooled)
        cos, sin = rope_tables(positions[:G * r:r], self.rd, self.theta)
        return rope_tail(pooled.unsqueeze(1), cos, sin, self.rd)[:, 0]


class V4Indexer(nn.Module):
    """Scores compressed groups per query: sum_h w[t, h] * relu(q[t, h] . k[g]), best ``index_topk``."""

    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__()
        x = cfg.extra
        self.Hi, self.Di, self.topk = int(x.get("index_n_heads", 64)), int(x.get("index_head_dim", 128)), int(x.get("index_topk", 512))
        self.rd = x["qk_rope_head_dim"]
        self.theta = float(x.get("compress_rope_theta", cfg.rope_theta))
        self.linear_wq_b = Linear(x["q_lora_rank"], self.Hi * self.Di, dtype=dtype, device=device)
        self.linear_weights_proj = Linear(cfg.hidden_size, self.Hi, dtype=dtype, device=device)
        self.compressor = Compressor(cfg, self.Di, 4, dtype=dtype, device=device)

    @torch.no_grad()
    def forward(self, x, qr, positions) -> torch.Tensor:
        """One document -> boolean [L, G]: groups each query keeps (before the causal cut)."""
        L = x.shape[0]
        k = self.compressor(x, positions)
        G = k.shape[0]
        if G <= self.topk:
            return torch.ones(L, G, dtype=torch.bool, device=x.device)
        cos, sin = rope_tables(positions, self.rd, self.theta)
        q = rope_tail(self.linear_wq_b(qr).view(L, self.Hi, self.Di), cos, sin, self.rd)
        w = self.linear_weights_proj(x).float() * (self.Hi ** -0.5) * (self.Di ** -0.5)
        s = torch.einsum("thg,th->tg", torch.relu(torch.einsum("thd,gd->thg", q.float(), k.float())), w)
        visible = torch.arange(G, device=x.device).view(1, G) < ((positions - positions[0] + 1) // 4).view(L, 1)
        s = s.masked_fill(~visible, float("-inf"))
        return torch.zeros(L, G, dtype=torch.bool, device=x.device).scatter_(1, s.topk(self.topk, dim=-1).indices, True)


class V4Attention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        x = cfg.extra
        self.H, self.hd, self.rd = cfg.num_attention_heads, cfg.extra["v4_head_dim"], x["qk_rope_head_dim"]
        self.G, self.r_o = int(x.get("o_groups", 1)), int(x["o_lora_rank"])
        self.window = int(cfg.sliding_window or 128)
        ratios = x.get("compress_ratios")
        self.ratio = int(ratios[layer_idx]) if ratios else 0
        self.theta = float(x.get("compress_rope_theta", cfg.rope_theta)) if self.ratio else float(cfg.rope_theta)
        self.eps = cfg.rms_norm_eps
        hs = cfg.hidden_size
        self.attn_sink = nn.Parameter(torch.zeros(self.H, dtype=torch.float32, device=device))
        self.wq_a = Linear(hs, x["q_lora_rank"], dtype=dtype, device=device)
        self.q_norm = RMSNorm(x["q_lora_rank"], self.eps, dtype=dtype, device=device)
        self.wq_b = Linear(x["q_lora_rank"], self.H * self.hd, dtype=dtype, device=device)
        self.wkv = Linear(hs, self.hd, dtype=dtype, device=device)
        self.kv_norm = RMSNorm(self.hd, self.eps, dtype=dtype, device=device)
        self.wo_a = Linear(self.H * self.hd // self.G, self.G * self.r_o, dtype=dtype, device=device)
        self.wo_b = Linear(self.G * self.r_o, hs, dtype=dtype, device=device)
        self.scale = self.hd ** -0.5
        self.compressor = Compressor(cfg, self.hd, self.ratio, dtype=dtype, device=device) if self.ratio else None
        self.indexer = V4Indexer(cfg, dtype=dtype, device=device) if self.ratio == 4 else None

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T = x.shape[0]
        pos = ctx.position_ids
        cos, sin = rope_tables(pos, self.rd, self.theta)
        qr = self.q_norm(self.wq_a(x))
        q = self.wq_b(qr).view(T, self.H, self.hd).float()
        q = (q * torch.rsqrt(q.square().mean(-1, keepdim=True) + self.eps)).to(x.dtype)
        q = rope_tail(q, cos, sin, self.rd)
        kv = rope_tail(self.kv_norm(self.wkv(x)).unsqueeze(1), cos, sin, self.rd)[:, 0]            # [T, hd]
        outs = []
        cu = ctx.cu_seqlens.tolist()
        sink = self.attn_sink.float().view(self.H, 1, 1)
        for s, e in zip(cu[:-1], cu[1:]):
            L = e - s
            if L <= 0:
                continue
            t = torch.arange(L, device=x.device)
            keys = kv[s:e]
            allow = (t.view(L, 1) >= t.view(1, L)) & (t.view(L, 1) - t.view(1, L) < self.window)
            if self.compressor is not None:
                ck = self.compressor(x[s:e], pos[s:e])
                Gc = ck.shape[0]
                if Gc:
                    vis = torch.arange(Gc, device=x.device).view(1, Gc) < ((t + 1) // self.ratio).view(L, 1)
                    if self.indexer is not None:
                        vis = vis & self.indexer(x[s:e].detach(), qr[s:e].detach(), pos[s:e])
                    keys = torch.cat([keys, ck], 0)
                    allow = torch.cat([allow, vis], 1)
            logits = torch.einsum("thd,kd->htk", q[s:e].float(), keys.float()) * self.scale
            logits = logits.masked_fill(~allow.unsqueeze(0), float("-inf"))
            m = torch.maximum(logits.amax(-1, keepdim=True), sink)
            p = torch.exp(logits - m)
            p = p / (p.sum(-1, keepdim=True) + torch.exp(sink - m))
            outs.append(torch.einsum("htk,kd->thd", p, keys.float()).to(x.dtype))
        if cu[-1] < T:
            outs.append(x.new_zeros(T - cu[-1], self.H, self.hd))
        o = rope_tail(torch.cat(outs, 0), cos, sin, self.rd, inverse=True)
        o = o.reshape(T, self.G, self.H // self.G * self.hd)
        w = self.wo_a.weight.view(self.G, self.r_o, -1)
        return self.wo_b(torch.einsum("tgd,grd->tgr", o, w).reshape(T, self.G * self.r_o))


# ------------------------------------------------------------------------------------------------
# MoE: sqrt(softplus) scores; the first ``num_hash_layers`` layers pick experts from a token-id table
# ------------------------------------------------------------------------------------------------
class V4MoE(MoEBlock):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__(cfg, layer_idx, dtype=dtype, device=device)
        self.is_hash_layer = layer_idx < int(cfg.extra.get("num_hash_layers", 0))
        if self.is_hash_layer:
            self.gate.e_score_correction_bias = None
            # frozen token-id -> expert-ids table, kept as a (non-trainable) floating-point parameter so
            # that it is sharded, gathered and checkpointed with the other weights; expert ids up to
            # 256 are exact in bf16
            self.tid2eid = nn.Parameter(torch.zeros(cfg.vocab_size, cfg.num_experts_per_tok, dtype=dtype,
                                                    device=device), requires_grad=False)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        if self.is_hash_layer and ("routing_replay", self.layer_idx) not in ctx.aux:
            ids = ctx.aux.get("input_ids")
            if ids is None:
                raise ValueError("hash-routed layers need the token ids (ctx.aux['input_ids'])")
            ctx.aux[("routing_replay", self.layer_idx)] = self.tid2eid[ids.reshape(-1)].round().long()
            try:
                return super().forward(x, ctx)
            finally:
                ctx.aux.pop(("routing_replay", self.layer_idx), None)
        return super().forward(x, ctx)


def init_hash_table_(table: torch.Tensor, num_experts: int, gen: torch.Generator) -> None:
    """Fixed pseudo-random token -> experts table (k distinct experts per token id)."""
    V, k = table.shape
    table.copy_(torch.rand(V, num_experts, generator=gen).topk(k, dim=-1).indices.to(table.dtype))


class V4Layer(nn.Module):
    """Activations between layers are (stream [T, hc, H], None)."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.self_attn = V4Attention(cfg, layer_idx, dtype=dtype, device=device)
        self.mlp = V4MoE(cfg, layer_idx, dtype=dtype, device=device) if cfg.layer_is_moe(layer_idx) else \
            MLP(cfg.hidden_size, cfg.intermediate_size, dtype=dtype, device=device, tensor_parallel=False,
                swiglu_limit=cfg.extra.get("dense_swiglu_limit"))
        self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, dtype=dtype, device=device)
        self.hc_attn = HyperConnection(cfg, device=device)
        self.hc_ffn = HyperConnection(cfg, device=device)

    def forward(self, x: torch.Tensor, residual: Optional[torch.Tensor], ctx: StepContext):
        h, post, comb = self.hc_attn.pre(x)
        x = HyperConnection.post(self.self_attn(self.input_layernorm(h), ctx), x, post, comb)
        h, post, comb = self.hc_ffn.pre(x)
        h = self.post_attention_layernorm(h)
        y = self.mlp(h, ctx) if isinstance(self.mlp, MoEBlock) else self.mlp(h)
        return HyperConnection.post(y, x, post, comb), None
