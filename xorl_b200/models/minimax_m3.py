"""MiniMax-M3 text model pieces: attention whose sparse layers carry an index projection for
block-sparse key selection, on top of the shared decoder (zero-centred norms, per-head q/k norm
weights, partial rotary embedding, sigmoid-routed MoE with clamped SwiGLU experts and a shared
expert; src/xorl/models/transformers/minimax_m3/modeling_minimax_m3.py).

Training runs dense causal attention on every layer, as the reference does (its sparse path has no
backward, src/xorl/models/transformers/minimax_m3/msa_attention.py:66-70).  ``msa_attention`` is the
block-sparse inference path: every query scores key blocks with its index head (the maximum index
logit over the block's visible keys), keeps the ``topk_blocks`` best including the forced first
and most recent blocks, and attends to those blocks only.
"""
from __future__ import annotations

import torch

from ..ops import attention as attn_ops
from .config import ModelConfig
from .context import StepContext
from .layers import Attention, Linear, RMSNorm, per_head_rmsnorm


def msa_attention(q, k, v, iq, ik, cu_seqlens, scale, *, block_size: int, topk_blocks: int,
                  force_begin_blocks: int = 0, force_end_blocks: int = 1) -> torch.Tensor:
    """q [T,Hq,D], k/v [T,Hkv,D], iq/ik [T,Hi,Di] -> [T,Hq,D].  Query heads share the selection of
    index head ``h * Hi // Hq``; selection and attention are causal inside each document."""
    T, Hq, D = q.shape
    Hkv, Hi = k.shape[1], iq.shape[1]
    out = torch.empty(T, Hq, v.shape[-1], dtype=q.dtype, device=q.device)
    cu = cu_seqlens.tolist()
    iscale = iq.shape[-1] ** -0.5
    for b in range(len(cu) - 1):
        s, e = cu[b], cu[b + 1]
        L = e - s
        if L <= 0:
            continue
        nb = (L + block_size - 1) // block_size
        pos = torch.arange(L, device=q.device)
        blk = pos // block_size
        causal = pos.view(L, 1) >= pos.view(1, L)                                  # [Lq, Lk]
        logits = torch.einsum("qhd,khd->hqk", iq[s:e].float(), ik[s:e].float()) * iscale
        logits = logits.masked_fill(~causal, float("-inf"))
        pad = nb * block_size - L
        if pad:
            logits = torch.nn.functional.pad(logits, (0, pad), value=float("-inf"))
        score = logits.view(Hi, L, nb, block_size).amax(-1)                        # [Hi, Lq, nb]
        qb = blk.view(1, L, 1)
        bidx = torch.arange(nb, device=q.device).view(1, 1, nb)
        forced = (bidx < force_begin_blocks) | ((bidx <= qb) & (bidx > qb - force_end_blocks))
        score = torch.where(forced & (bidx <= qb), torch.full_like(score, float("inf")), score)
        kk = min(topk_blocks, nb)
        top = score.topk(kk, dim=-1).indices                                       # [Hi, Lq, kk]
        keep_blk = torch.zeros(Hi, L, nb, dtype=torch.bool, device=q.device).scatter_(-1, top, True)
        keep_blk &= score > float("-inf")                                          # never a future block
        keep = keep_blk[:, :, blk] & causal.unsqueeze(0)                           # [Hi, Lq, Lk]
        keep_h = keep.repeat_interleave(Hq // Hi, dim=0)                           # [Hq, Lq, Lk]
        kh = k[s:e].float().repeat_interleave(Hq // Hkv, dim=1)
        vh = v[s:e].float().repeat_interleave(Hq // Hkv, dim=1)
        att = torch.einsum("qhd,khd->hqk", q[s:e].float(), kh) * scale
        att = att.masked_fill(~keep_h, float("-inf")).softmax(-1)
        out[s:e] = torch.einsum("hqk,khd->qhd", att, vh).to(q.dtype)
    return out


class MiniMaxAttention(Attention):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__(cfg, layer_idx, dtype=dtype, device=device)
        x = cfg.extra
        freq = x.get("sparse_attention_freq") or []
        self.is_sparse_layer = bool(freq[layer_idx]) if layer_idx < len(freq) else False
        self.block_size = int(x.get("sparse_block_size", 128))
        self.topk_blocks = int(x.get("sparse_topk_blocks", 16))
        self.begin_blocks = int(x.get("sparse_init_block", 0))
        self.local_blocks = int(x.get("sparse_local_block", 1))
        if self.is_sparse_layer:
            self.Hi = int(x.get("sparse_num_index_heads", 4))
            self.Di = int(x.get("sparse_index_dim", cfg.head_dim))
            H = cfg.hidden_size
            self.index_q_proj = Linear(H, self.Hi * self.Di, bias=cfg.attention_bias, dtype=dtype, device=device)
            self.index_k_proj = Linear(H, self.Hi * self.Di, bias=cfg.attention_bias, dtype=dtype, device=device)
            zc = cfg.zero_centered_norm
            self.index_q_norm = RMSNorm(self.Hi * self.Di, cfg.rms_norm_eps, zc, dtype, device)
            self.index_k_norm = RMSNorm(self.Hi * self.Di, cfg.rms_norm_eps, zc, dtype, device)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        if not (self.is_sparse_layer and ctx.aux.get("minimax_msa") and not torch.is_grad_enabled()):
            return super().forward(x, ctx)
        T = x.shape[0]
        q, k, v = self._qkv_heads(self.qkv_proj(x), ctx)
        iq = per_head_rmsnorm(self.index_q_proj(x).view(T, self.Hi, self.Di), self.index_q_norm.weight,
                              self.index_q_norm.eps, self.index_q_norm.zero_centered)
        ik = per_head_rmsnorm(self.index_k_proj(x).view(T, self.Hi, self.Di), self.index_k_norm.weight,
                              self.index_k_norm.eps, self.index_k_norm.zero_centered)
        rot = ctx.cos.shape[-1] * 2
        iq = torch.cat([attn_ops.rope_reference(iq[..., :rot], ctx.cos, ctx.sin), iq[..., rot:]], -1)
        ik = torch.cat([attn_ops.rope_reference(ik[..., :rot], ctx.cos, ctx.sin), ik[..., rot:]], -1)
        out = msa_attention(q, k, v, iq, ik, ctx.cu_seqlens, self.scale, block_size=self.block_size,
                            topk_blocks=self.topk_blocks, force_begin_blocks=self.begin_blocks,
                            force_end_blocks=self.local_blocks)
        return self.o_proj(out.reshape(T, self.Hq * self.D))
