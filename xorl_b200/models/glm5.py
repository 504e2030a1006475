"""GLM-5 (``glm_moe_dsa``): multi-head latent attention restricted to the keys chosen by a
"lightning indexer", plus the DeepSeek-style sigmoid-routed MoE of the shared decoder.

Indexer (src/xorl/models/transformers/glm5/indexer.py): ``index_q = wq_b(q_compressed)``
``[T, Hi, Di]`` from the compressed query that multi-head latent attention already computes,
one ``index_k = LayerNorm(wk(x))`` ``[T, Di]`` per token, head gates ``weights_proj(x) * Hi^-1/2``;
rotary embedding on the first ``qk_rope_head_dim`` channels of both;

    score[t, s] = sum_h gate[t, h] * relu(index_q[t, h] . index_k[s]) * Di^-1/2      (s <= t, same document)

and every query keeps its ``index_topk`` best keys.  The selection carries no gradient.  Layers
without an indexer of their own (``index_topk_freq`` > 1) reuse the selection of the closest
earlier layer that has one (src/xorl/models/transformers/glm5/index_share.py).
"""
from __future__ import annotations

from typing import List

import torch
from torch import nn

from ..ops import attention as attn_ops
from .config import ModelConfig
from .context import StepContext
from .layers import Linear
from .mla import MLAttention


def layer_has_indexer(cfg: ModelConfig, layer_idx: int) -> bool:
    x = cfg.extra
    pattern = x.get("index_topk_pattern")
    if pattern:
        return bool(pattern[layer_idx])
    freq = max(1, int(x.get("index_topk_freq", 1)))
    off = int(x.get("index_skip_topk_offset", 0))
    return layer_idx < off or (layer_idx - off) % freq == 0


def indexer_scores(index_q: torch.Tensor, index_k: torch.Tensor, gates: torch.Tensor) -> torch.Tensor:
    """index_q [L, Hi, Di], index_k [L, Di], gates [L, Hi] -> scores [L, L] (fp32, no mask)."""
    dots = torch.einsum("qhd,kd->qhk", index_q.float(), index_k.float())
    return torch.einsum("qhk,qh->qk", torch.relu(dots), gates.float()) * index_q.shape[-1] ** -0.5


def select_topk_keys(scores: torch.Tensor, topk: int) -> torch.Tensor:
    """Boolean [L, L]: the ``topk`` best causal keys of every query (all of them when fewer exist)."""
    L = scores.shape[0]
    causal = torch.ones(L, L, dtype=torch.bool, device=scores.device).tril()
    if topk >= L:
        return causal
    s = scores.masked_fill(~causal, float("-inf"))
    idx = s.topk(topk, dim=-1).indices
    keep = torch.zeros_like(causal).scatter_(-1, idx, True)
    return keep & causal


class DsaIndexer(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__()
        x = cfg.extra
        self.Hi, self.Di = int(x.get("index_n_heads", 32)), int(x.get("index_head_dim", 128))
        self.topk = int(x.get("index_topk", 2048))
        self.d_rope = x["qk_rope_head_dim"]
        self.interleaved = bool(x.get("indexer_rope_interleave", True))
        self.wq_b = Linear(x["q_lora_rank"], self.Hi * self.Di, dtype=dtype, device=device)
        self.wk = Linear(cfg.hidden_size, self.Di, dtype=dtype, device=device)
        self.k_norm_weight = nn.Parameter(torch.ones(self.Di, dtype=dtype, device=device))
        self.k_norm_bias = nn.Parameter(torch.zeros(self.Di, dtype=dtype, device=device))
        self.weights_proj = Linear(cfg.hidden_size, self.Hi, dtype=dtype, device=device)

    def _rope(self, t, cos, sin):
        T, h, d = t.shape
        if self.interleaved:
            t = t.view(T, h, d // 2, 2).transpose(-1, -2).reshape(T, h, d)
        return attn_ops.rope_reference(t, cos, sin)

    @torch.no_grad()
    def select(self, x: torch.Tensor, q_compressed: torch.Tensor, ctx: StepContext) -> List[torch.Tensor]:
        """One boolean keep-matrix [L, L] per document."""
        T = x.shape[0]
        iq = self.wq_b(q_compressed).view(T, self.Hi, self.Di)
        ik = torch.nn.functional.layer_norm(self.wk(x).float(), (self.Di,), self.k_norm_weight.float(),
                                            self.k_norm_bias.float(), 1e-6).to(x.dtype)
        gates = self.weights_proj(x).float() * self.Hi ** -0.5
        r = self.d_rope
        iq = torch.cat([self._rope(iq[..., :r], ctx.cos, ctx.sin), iq[..., r:]], -1)
        ik = torch.cat([self._rope(ik[:, None, :r], ctx.cos, ctx.sin)[:, 0], ik[:, r:]], -1)
        cu = ctx.cu_seqlens.tolist()
        return [select_topk_keys(indexer_scores(iq[s:e], ik[s:e], gates[s:e]), self.topk)
                for s, e in zip(cu[:-1], cu[1:])]


class Glm5Attention(MLAttention):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__(cfg, layer_idx, dtype=dtype, device=device)
        if not self.q_lora:
            raise ValueError("the sparse indexer reads the compressed query: q_lora_rank is required")
        self.has_indexer = layer_has_indexer(cfg, layer_idx)
        self.indexer = DsaIndexer(cfg, dtype=dtype, device=device) if self.has_indexer else None
        self.producer = max(i for i in range(layer_idx + 1) if layer_has_indexer(cfg, i)) \
            if any(layer_has_indexer(cfg, i) for i in range(layer_idx + 1)) else None

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T = x.shape[0]
        qc = self.q_a_layernorm(self.q_a_proj(x))
        key = ("dsa_keep", self.producer)
        if self.has_indexer and key not in ctx.aux:
            # computed once per micro-batch: a recomputed forward and the layers that share this
            # layer's selection read the stored matrices
            ctx.aux[key] = self.indexer.select(x.detach(), qc.detach(), ctx)
        keep = ctx.aux.get(key)
        q = self.q_b_proj(qc).view(T, self.H, self.d_qk)
        q_nope, q_rope = q.split([self.d_nope, self.d_rope], dim=-1)
        ckv = self.kv_a_proj_with_mqa(x)
        c, k_rope = ckv.split([self.kv_lora, self.d_rope], dim=-1)
        kv = self.kv_b_proj(self.kv_a_layernorm(c)).view(T, self.H, self.d_nope + self.d_v)
        k_nope, v = kv.split([self.d_nope, self.d_v], dim=-1)
        q_rope = self._rope(q_rope, ctx.cos, ctx.sin)
        k_rope = self._rope(k_rope.reshape(T, 1, self.d_rope), ctx.cos, ctx.sin).expand(T, self.H, self.d_rope)
        qf = torch.cat([q_nope, q_rope], -1)
        kf = torch.cat([k_nope, k_rope], -1)
        if keep is None:
            out = attn_ops.attention_reference(qf, kf, v.contiguous(), ctx.cu_seqlens, ctx.causal, self.scale)
        else:
            out = torch.empty(T, self.H, self.d_v, dtype=x.dtype, device=x.device)
            cu = ctx.cu_seqlens.tolist()
            pieces = []
            for m, (s, e) in zip(keep, zip(cu[:-1], cu[1:])):
                att = torch.einsum("qhd,khd->hqk", qf[s:e].float(), kf[s:e].float()) * self.scale
                att = att.masked_fill(~m.unsqueeze(0), float("-inf")).softmax(-1)
                pieces.append(torch.einsum("hqk,khd->qhd", att, v[s:e].float()).to(x.dtype))
            if cu[-1] < T:
                pieces.append(torch.zeros(T - cu[-1], self.H, self.d_v, dtype=x.dtype, device=x.device))
            out = torch.cat(pieces, 0)
        return self.o_proj(out.reshape(T, self.H * self.d_v))
