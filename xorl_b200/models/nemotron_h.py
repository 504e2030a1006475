"""Nemotron-H: a stack of single-mixer blocks ``x = x + mixer(norm(x))`` whose mixer is a Mamba2
state-space layer, a rotary-free GQA attention layer or a latent mixture of experts, chosen per
layer by ``layers_block_type`` (src/xorl/models/transformers/nemotron_h/modeling_nemotron_h.py).

The MoE layer routes with sigmoid scores (group-limited, selection-only correction bias), projects
tokens to a latent width, runs non-gated relu-squared experts there, projects back, and adds a
non-gated shared expert computed from the unprojected input.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..ops import moe as moe_ops
from .config import ModelConfig
from .context import StepContext
from .layers import Attention, Linear, RMSNorm
from .mamba2 import Mamba2Mixer
from .moe import Experts, MoEBlock


class ReluSquaredMLP(nn.Module):
    """down(relu(up(x))^2)."""

    def __init__(self, hidden: int, intermediate: int, bias: bool = False, dtype=None, device=None):
        super().__init__()
        self.up_proj = Linear(hidden, intermediate, bias=bias, dtype=dtype, device=device)
        self.down_proj = Linear(intermediate, hidden, bias=bias, dtype=dtype, device=device)

    def forward(self, x):
        return self.down_proj(torch.relu(self.up_proj(x)).square())


class NemotronHMoE(MoEBlock):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__(cfg, layer_idx, dtype=dtype, device=device)
        x = cfg.extra
        latent = x.get("moe_latent_size") or cfg.hidden_size
        self.fc1_latent_proj = Linear(cfg.hidden_size, latent, bias=cfg.mlp_bias, dtype=dtype, device=device)
        self.fc2_latent_proj = Linear(latent, cfg.hidden_size, bias=cfg.mlp_bias, dtype=dtype, device=device)
        self.shared_expert = ReluSquaredMLP(cfg.hidden_size, x.get("moe_shared_expert_intermediate_size")
                                            or cfg.moe_intermediate_size, cfg.mlp_bias, dtype, device)

    def build_experts(self, cfg, dtype, device):
        return Experts(cfg, self.num_local, dtype=dtype, device=device,
                       hidden=cfg.extra.get("moe_latent_size") or cfg.hidden_size, gated=False, activation="relu2")

    def pre_experts(self, x):
        return self.fc1_latent_proj(x)

    def post_experts(self, y):
        return self.fc2_latent_proj(y)


class NemotronHLayer(nn.Module):
    """One block.  Activations between blocks are the pair (mixer output, residual stream before
    it), like the other decoder layers, so the norm runs fused with the residual add."""

    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.block_type = cfg.extra["layers_block_type"][layer_idx]
        self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, False, dtype, device)
        if self.block_type == "mamba":
            self.mixer = Mamba2Mixer(cfg, layer_idx, dtype=dtype, device=device)
        elif self.block_type == "attention":
            self.mixer = Attention(cfg, layer_idx, dtype=dtype, device=device)
        elif self.block_type == "moe":
            self.mixer = NemotronHMoE(cfg, layer_idx, dtype=dtype, device=device)
        elif self.block_type == "mlp":
            self.mixer = ReluSquaredMLP(cfg.hidden_size, cfg.intermediate_size, cfg.mlp_bias, dtype, device)
        else:
            raise ValueError(f"unknown layers_block_type entry {self.block_type!r}")

    def forward(self, h: torch.Tensor, residual: Optional[torch.Tensor], ctx: StepContext):
        if residual is None:
            y, x = self.norm(h), h
        else:
            y, x = self.norm(h, residual=residual)
        if self.block_type == "mlp":
            return self.mixer(y), x
        return self.mixer(y, ctx), x
