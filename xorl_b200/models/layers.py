"""Building blocks of the decoder families: RMSNorm, linear, fused-qkv attention, SwiGLU MLP.

Modules own parameters only; the math is in ``xorl_b200.ops`` (sm_100a kernels on CUDA, PyTorch on
CPU).  Parameter names follow the reference's fused layout (``self_attn.qkv_proj``,
``mlp.gate_up_proj``; src/xorl/models/layers/attention/multi_head_attention.py:15-189,
src/xorl/models/transformers/qwen3/modeling_qwen3.py:40-81) so checkpoints interchange.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
from torch import nn

from ..ops import activation as act_ops
from ..ops import attention as attn_ops
from ..ops import gemm as gemm_ops
from ..ops import norm as norm_ops
from .config import ModelConfig
from .context import StepContext


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float = 1e-6, zero_centered: bool = False, dtype=None,
                 device=None):
        super().__init__()
        init = torch.zeros if zero_centered else torch.ones
        self.weight = nn.Parameter(init(dim, dtype=dtype, device=device))
        self.eps = eps
        self.zero_centered = zero_centered

    def forward(self, x, residual=None):
        return norm_ops.rmsnorm(x, self.weight, self.eps, residual=residual,
                                zero_centered=self.zero_centered)


class Linear(nn.Module):
    """Weight ``[out, in]`` (+ optional bias); forward through the tcgen05 GEMM."""

    def __init__(self, in_features: int, out_features: int, bias: bool = False, dtype=None,
                 device=None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(out_features, dtype=dtype, device=device)) if bias else None

    def forward(self, x):
        return gemm_ops.linear(x, self.weight, self.bias)


def per_head_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, zero_centered: bool) -> torch.Tensor:
    """x [T, heads, D], weight [heads * D]: RMS over D, one weight vector per head."""
    h = x.float()
    h = h * torch.rsqrt(h.pow(2).mean(-1, keepdim=True) + eps)
    w = weight.float().view(x.shape[1], x.shape[2])
    return (h * (1.0 + w if zero_centered else w)).to(x.dtype)


def _tp():
    from ..parallel.tp import tp_info
    return tp_info()


def _sp():
    """The sequence-parallel tensor-parallel context, or None (plain TP with all-reduces)."""
    from ..parallel.state import get_parallel_state
    if not get_parallel_state().tp_sequence_parallel:
        return None
    from ..parallel.tp_fused import sp_context
    return sp_context()


class Attention(nn.Module):
    """Fused qkv projection -> (per-head qk RMSNorm) -> RoPE -> varlen causal attention -> o_proj.
    A context-parallel strategy on ``ctx.cp`` takes over the middle part when present."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        self.Hq, self.Hkv, self.D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
        H = cfg.hidden_size
        self.tp, self.tp_rank, self.tp_group = _tp()
        self.sp = _sp() if self.tp > 1 else None
        if self.tp > 1:
            if self.Hq % self.tp or self.Hkv % self.tp:
                raise ValueError(f"heads ({self.Hq}, {self.Hkv}) not divisible by tensor_parallel_size {self.tp}")
            fq, fkv = self.Hq * self.D, self.Hkv * self.D
            self.Hq //= self.tp
            self.Hkv //= self.tp
        self.qkv_proj = Linear(H, (self.Hq + 2 * self.Hkv) * self.D, bias=cfg.attention_bias,
                               dtype=dtype, device=device)
        self.o_proj = Linear(self.Hq * self.D, H, bias=False, dtype=dtype, device=device)
        if self.tp > 1:
            from ..parallel.tp import mark_col, mark_row
            mark_col(self.qkv_proj.weight, (fq + 2 * fkv, H), (fq, fkv, fkv))
            if self.qkv_proj.bias is not None:
                mark_col(self.qkv_proj.bias, (fq + 2 * fkv,), (fq, fkv, fkv))
            mark_row(self.o_proj.weight, (H, fq))
        self.use_qk_norm = cfg.use_qk_norm
        if cfg.use_qk_norm:
            nd = self.D if not cfg.qk_norm_full else None
            # MiniMax-M3: every head has its own norm weights (statistics still per head)
            self.qk_norm_per_head = bool(cfg.extra.get("qk_norm_per_head_weights"))
            if self.qk_norm_per_head:
                nd = None
            zc = cfg.zero_centered_norm and self.qk_norm_per_head
            self.q_norm = RMSNorm(nd or self.Hq * self.D, cfg.rms_norm_eps, zc, dtype=dtype, device=device)
            self.k_norm = RMSNorm(nd or self.Hkv * self.D, cfg.rms_norm_eps, zc, dtype=dtype, device=device)
            if self.tp > 1 and not cfg.qk_norm_full:
                # every TP rank sees only its own heads: gradients are summed over the TP group
                self.q_norm.weight._xb_tp_reduce = True
                self.k_norm.weight._xb_tp_reduce = True
        self.scale = 1.0 / math.sqrt(self.D)
        self.no_rope = bool(cfg.extra.get("no_rope"))       # Nemotron-H attention has no positional embedding
        self.window = cfg.sliding_window if (cfg.layer_types is None or
                                            cfg.layer_types[layer_idx] == "sliding_attention") else None
        # Qwen3-Next / Qwen3.5: the attention output is multiplied by sigmoid(gate(x)) before o_proj
        self.out_gate = Linear(H, self.Hq * self.D, dtype=dtype, device=device) \
            if cfg.extra.get("attn_output_gate") else None
        if self.out_gate is not None and self.tp > 1:
            from ..parallel.tp import mark_col
            mark_col(self.out_gate.weight, (self.Hq * self.tp * self.D, H), (self.Hq * self.tp * self.D,))
        self.sinks = nn.Parameter(torch.zeros(self.Hq, dtype=dtype, device=device)) if cfg.attention_sinks else None
        if self.sinks is not None and self.tp > 1:
            from ..parallel.tp import mark_col
            mark_col(self.sinks, (self.Hq * self.tp,), (self.Hq * self.tp,))

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        if self.sp is not None:
            # x holds this rank's tokens: the all-gather runs inside the projection's GEMM kernel
            from ..parallel.tp_fused import gather_tokens, sp_column_linear
            qkv = sp_column_linear(x, self.qkv_proj.weight, self.qkv_proj.bias, self.sp)
            if self.out_gate is not None:
                x = gather_tokens(x, self.sp)
        else:
            if self.tp > 1:
                from ..parallel.tp import copy_to_tp
                x = copy_to_tp(x, self.tp_group)
            qkv = self.qkv_proj(x)
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        if ctx.cp is not None:
            out = ctx.cp.attention(self, qkv, ctx)
        elif (self.cfg.qk_norm_full or self.cfg.partial_rotary_factor != 1.0 or self.window
              or self.sinks is not None or self.no_rope or getattr(self, "qk_norm_per_head", False)):
            out = self._unfused_attention(qkv, ctx)
        else:
            wq = self.q_norm.weight if self.use_qk_norm else None
            wk = self.k_norm.weight if self.use_qk_norm else None
            out = attn_ops.qk_norm_rope_attention(qkv, wq, wk, ctx.cos, ctx.sin, ctx.cu_seqlens,
                                                  Hq, Hkv, D, self.cfg.rms_norm_eps, ctx.causal,
                                                  self.scale)
        if self.out_gate is not None:
            out = out * torch.sigmoid(self.out_gate(x).float()).to(out.dtype)
        if self.sp is not None:
            from ..parallel.tp_fused import sp_row_linear
            return sp_row_linear(out, self.o_proj.weight, None, self.sp)
        out = self.o_proj(out)
        if self.tp > 1:
            from ..parallel.tp import reduce_from_tp
            out = reduce_from_tp(out, self.tp_group)
        return out

    def _unfused_attention(self, qkv, ctx):
        """General path (whole-projection qk-norm, partial rotary): separate ops."""
        q, k, v = self._qkv_heads(qkv, ctx)
        T, Hq, D = q.shape
        # sliding windows and sink logits are features of the tcgen05 kernel (masked softmax on CPU)
        out = attn_ops.flash_attn_varlen(q, k, v, ctx.cu_seqlens, ctx.causal, self.scale,
                                         window=self.window, sinks=self.sinks)
        return out.reshape(T, Hq * D)

    def _qkv_heads(self, qkv, ctx):
        """Fused projection output -> normalised, rotated q [T, Hq, D], k, v [T, Hkv, D]."""
        T = qkv.shape[0]
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        if self.use_qk_norm and self.cfg.qk_norm_full:
            q, k = self.q_norm(q), self.k_norm(k)
        q, k, v = q.reshape(T, Hq, D), k.reshape(T, Hkv, D), v.reshape(T, Hkv, D)
        if self.use_qk_norm and getattr(self, "qk_norm_per_head", False):
            q = per_head_rmsnorm(q, self.q_norm.weight, self.q_norm.eps, self.q_norm.zero_centered)
            k = per_head_rmsnorm(k, self.k_norm.weight, self.k_norm.eps, self.k_norm.zero_centered)
        elif self.use_qk_norm and not self.cfg.qk_norm_full:
            q = self.q_norm(q.reshape(T * Hq, D)).reshape(T, Hq, D)
            k = self.k_norm(k.reshape(T * Hkv, D)).reshape(T, Hkv, D)
        rot = ctx.cos.shape[-1] * 2
        if self.no_rope:
            pass
        elif rot == D:
            q, k = attn_ops.rope_reference(q, ctx.cos, ctx.sin), attn_ops.rope_reference(k, ctx.cos, ctx.sin)
        else:
            q = torch.cat([attn_ops.rope_reference(q[..., :rot], ctx.cos, ctx.sin), q[..., rot:]], -1)
            k = torch.cat([attn_ops.rope_reference(k[..., :rot], ctx.cos, ctx.sin), k[..., rot:]], -1)
        return q, k, v


class MLP(nn.Module):
    """SwiGLU feed-forward with a fused gate_up projection ``[2I, H]`` (gate rows first)."""

    def __init__(self, hidden: int, intermediate: int, bias: bool = False, dtype=None, device=None,
                 tensor_parallel: bool = True, swiglu_limit: Optional[float] = None):
        """``swiglu_limit``: clamped activation ``(up.clamp(+-l) + 1) * g * sigmoid(1.702 g)`` with
        ``g = gate.clamp(max=l)`` (MiniMax-M3) instead of SwiGLU."""
        super().__init__()
        self.swiglu_limit = swiglu_limit
        self.tp, self.tp_rank, self.tp_group = _tp() if tensor_parallel else (1, 0, None)
        self.sp = _sp() if self.tp > 1 else None
        full_I = intermediate
        if self.tp > 1:
            if intermediate % self.tp:
                raise ValueError(f"intermediate size {intermediate} not divisible by tp {self.tp}")
            intermediate //= self.tp
        self.gate_up_proj = Linear(hidden, 2 * intermediate, bias=bias, dtype=dtype, device=device)
        self.down_proj = Linear(intermediate, hidden, bias=bias, dtype=dtype, device=device)
        if self.tp > 1:
            from ..parallel.tp import mark_col, mark_row
            mark_col(self.gate_up_proj.weight, (2 * full_I, hidden), (full_I, full_I))
            mark_row(self.down_proj.weight, (hidden, full_I))

    def _act(self, h):
        if self.swiglu_limit is not None:
            from ..ops.moe import clamped_swiglu
            return clamped_swiglu(h, self.swiglu_limit)
        return act_ops.swiglu(h)

    def forward(self, x):
        if self.sp is not None:
            from ..parallel.tp_fused import sp_column_linear, sp_row_linear
            h = self._act(sp_column_linear(x, self.gate_up_proj.weight, self.gate_up_proj.bias, self.sp))
            y = sp_row_linear(h, self.down_proj.weight, None, self.sp)
            # a row-parallel bias is replicated: added once, after the reduction
            return y if self.down_proj.bias is None else y + self.down_proj.bias
        if self.tp > 1:
            from ..parallel.tp import copy_to_tp, reduce_from_tp
            x = copy_to_tp(x, self.tp_group)
            return reduce_from_tp(self.down_proj(self._act(self.gate_up_proj(x))), self.tp_group)
        return self.down_proj(self._act(self.gate_up_proj(x)))
