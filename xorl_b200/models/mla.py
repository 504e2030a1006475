"""Multi-head latent attention (DeepSeek-V3 family).

Queries and keys/values go through low-rank bottlenecks; every head's key is the concatenation of
a per-head "nope" part decoded from the shared latent and one rotary part shared by all heads
(src/xorl/models/transformers/deepseek_v3/modeling_deepseek_v3.py).  Head dimensions differ
between q/k (nope + rope, 192) and v (128), which the tcgen05 attention kernel (D = 128 for all
three) does not cover: the masked-softmax path computes it, padded-V flash attention is used when
the dimensions allow."""
from __future__ import annotations

import math

import torch
from torch import nn

from ..ops import attention as attn_ops
from .config import ModelConfig
from .context import StepContext
from .layers import Linear, RMSNorm


def _yarn_mscale(scale: float, mscale: float) -> float:
    return 1.0 if scale <= 1 else 0.1 * mscale * math.log(scale) + 1.0


class MLAttention(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        x = cfg.extra
        self.cfg, self.layer_idx = cfg, layer_idx
        self.H = cfg.num_attention_heads
        self.q_lora = x.get("q_lora_rank")
        self.kv_lora = x["kv_lora_rank"]
        self.d_nope, self.d_rope, self.d_v = x["qk_nope_head_dim"], x["qk_rope_head_dim"], x["v_head_dim"]
        self.d_qk = self.d_nope + self.d_rope
        hs, eps = cfg.hidden_size, cfg.rms_norm_eps
        if self.q_lora:
            self.q_a_proj = Linear(hs, self.q_lora, bias=cfg.attention_bias, dtype=dtype, device=device)
            self.q_a_layernorm = RMSNorm(self.q_lora, eps, dtype=dtype, device=device)
            self.q_b_proj = Linear(self.q_lora, self.H * self.d_qk, dtype=dtype, device=device)
        else:
            self.q_proj = Linear(hs, self.H * self.d_qk, dtype=dtype, device=device)
        self.kv_a_proj_with_mqa = Linear(hs, self.kv_lora + self.d_rope, bias=cfg.attention_bias,
                                         dtype=dtype, device=device)
        self.kv_a_layernorm = RMSNorm(self.kv_lora, eps, dtype=dtype, device=device)
        self.kv_b_proj = Linear(self.kv_lora, self.H * (self.d_nope + self.d_v), dtype=dtype, device=device)
        self.o_proj = Linear(self.H * self.d_v, hs, bias=cfg.attention_bias, dtype=dtype, device=device)
        self.scale = self.d_qk ** -0.5
        rs = cfg.rope_scaling or {}
        if rs.get("mscale_all_dim"):
            m = _yarn_mscale(rs.get("factor", 1.0), rs["mscale_all_dim"])
            self.scale *= m * m
        self.rope_interleaved = x.get("rope_interleave", True)

    def _rope(self, t, cos, sin):
        """t [T, h, d_rope].  DeepSeek stores rotary pairs interleaved; bring them to half-split
        order first so the shared rotate-half kernel applies."""
        if self.rope_interleaved:
            T, h, d = t.shape
            t = t.view(T, h, d // 2, 2).transpose(-1, -2).reshape(T, h, d)
        return attn_ops.rope_reference(t, cos, sin)

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T = x.shape[0]
        if self.q_lora:
            q = self.q_b_proj(self.q_a_layernorm(self.q_a_proj(x)))
        else:
            q = self.q_proj(x)
        q = q.view(T, self.H, self.d_qk)
        q_nope, q_rope = q.split([self.d_nope, self.d_rope], dim=-1)
        ckv = self.kv_a_proj_with_mqa(x)
        c, k_rope = ckv.split([self.kv_lora, self.d_rope], dim=-1)
        kv = self.kv_b_proj(self.kv_a_layernorm(c)).view(T, self.H, self.d_nope + self.d_v)
        k_nope, v = kv.split([self.d_nope, self.d_v], dim=-1)
        q_rope = self._rope(q_rope, ctx.cos, ctx.sin)
        k_rope = self._rope(k_rope.reshape(T, 1, self.d_rope), ctx.cos, ctx.sin).expand(T, self.H, self.d_rope)
        qf = torch.cat([q_nope, q_rope], -1)
        kf = torch.cat([k_nope, k_rope], -1)
        out = attn_ops.attention_reference(qf, kf, v.contiguous(), ctx.cu_seqlens, ctx.causal, self.scale)
        return self.o_proj(out.reshape(T, self.H * self.d_v))
