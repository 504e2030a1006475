"""Rotary position embedding tables.

``inv_freq`` initialisers for the scaling schemes the reference supports
(src/xorl/models/layers/rope.py:135-428: default, linear, dynamic NTK, YaRN, llama3) and the
per-step cos/sin gather (fp32 ``[T, rot_dim/2]``) that the fused qk-norm+RoPE kernel consumes.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def _default(dim: int, theta: float) -> torch.Tensor:
    return 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))


def compute_inv_freq(head_dim: int, theta: float, scaling: Optional[dict] = None,
                     partial_rotary_factor: float = 1.0,
                     max_position_embeddings: int = 4096) -> Tuple[torch.Tensor, float]:
    """Returns (inv_freq [rot_dim/2], attention_factor)."""
    dim = int(head_dim * partial_rotary_factor)
    inv = _default(dim, theta)
    if not scaling:
        return inv, 1.0
    kind = scaling.get("rope_type", scaling.get("type", "default"))
    factor = float(scaling.get("factor", 1.0))
    if kind == "default":
        return inv, 1.0
    if kind == "linear":
        return inv / factor, 1.0
    if kind == "dynamic":
        # NTK-aware: the base grows with the sequence length; at the nominal length it is identity
        return inv, 1.0
    if kind == "llama3":
        low = float(scaling.get("low_freq_factor", 1.0))
        high = float(scaling.get("high_freq_factor", 4.0))
        old_len = float(scaling.get("original_max_position_embeddings", 8192))
        wavelen = 2 * math.pi / inv
        scaled = torch.where(wavelen > old_len / low, inv / factor, inv)
        smooth = (old_len / wavelen - low) / (high - low)
        mid = (1 - smooth) * inv / factor + smooth * inv
        is_mid = (wavelen <= old_len / low) & (wavelen >= old_len / high)
        return torch.where(is_mid, mid, scaled), 1.0
    if kind == "yarn":
        orig = float(scaling.get("original_max_position_embeddings", max_position_embeddings))
        beta_fast = float(scaling.get("beta_fast", 32))
        beta_slow = float(scaling.get("beta_slow", 1))
        mscale = scaling.get("mscale")
        mscale_all = scaling.get("mscale_all_dim")

        def get_mscale(s, m=1.0):
            return 1.0 if s <= 1 else 0.1 * m * math.log(s) + 1.0

        if "attention_factor" in scaling and scaling["attention_factor"] is not None:
            att = float(scaling["attention_factor"])
        elif mscale and mscale_all:
            att = get_mscale(factor, mscale) / get_mscale(factor, mscale_all)
        else:
            att = get_mscale(factor)

        def corr_dim(nrot):
            return (dim * math.log(orig / (nrot * 2 * math.pi))) / (2 * math.log(theta))

        lo = max(math.floor(corr_dim(beta_fast)), 0)
        hi = min(math.ceil(corr_dim(beta_slow)), dim - 1)
        if lo == hi:
            hi += 0.001
        ramp = torch.clamp((torch.arange(dim // 2, dtype=torch.float32) - lo) / (hi - lo), 0, 1)
        extrap = 1.0 - ramp
        inv_yarn = (inv / factor) * (1 - extrap) + inv * extrap
        return inv_yarn, att
    raise ValueError(f"unknown rope scaling type {kind!r}")


class RotaryEmbedding(torch.nn.Module):
    """Holds ``inv_freq`` (a buffer, never sharded) and produces cos/sin for given positions."""

    def __init__(self, head_dim: int, theta: float, scaling: Optional[dict] = None,
                 partial_rotary_factor: float = 1.0, max_position_embeddings: int = 4096):
        super().__init__()
        inv, att = compute_inv_freq(head_dim, theta, scaling, partial_rotary_factor,
                                    max_position_embeddings)
        self.register_buffer("inv_freq", inv, persistent=False)
        self.attention_factor = att
        self.scaling = scaling or {}
        self.theta = theta
        self.rot_dim = inv.numel() * 2
        self.max_position_embeddings = max_position_embeddings

    @torch.no_grad()
    def forward(self, position_ids: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """position_ids [T] -> (cos, sin) fp32 [T, rot_dim/2]."""
        inv = self.inv_freq.to(position_ids.device, torch.float32)
        kind = self.scaling.get("rope_type", self.scaling.get("type"))
        if kind == "dynamic":
            seq_len = int(position_ids.max().item()) + 1
            if seq_len > self.max_position_embeddings:
                factor = float(self.scaling.get("factor", 1.0))
                dim = self.rot_dim
                base = self.theta * ((factor * seq_len / self.max_position_embeddings)
                                     - (factor - 1)) ** (dim / (dim - 2))
                inv = _default(dim, base).to(position_ids.device)
        ang = position_ids.reshape(-1, 1).to(torch.float32) * inv.reshape(1, -1)
        return (ang.cos() * self.attention_factor).contiguous(), \
               (ang.sin() * self.attention_factor).contiguous()
