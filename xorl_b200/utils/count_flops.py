"""Model FLOP estimates and device peak table for MFU, cf. src/xorl/utils/count_flops.py:50-78
(B200 2250e12, H100 989e12 dense bf16)."""
from __future__ import annotations

from typing import Sequence

import torch

DEVICE_PEAK_BF16 = {"B200": 2250e12, "GB200": 2500e12, "H200": 989e12, "H100": 989e12,
                    "H800": 989e12, "A100": 312e12, "A800": 312e12, "L40S": 362e12}


def get_device_flops(name: str | None = None) -> float:
    if name is None:
        name = torch.cuda.get_device_name() if torch.cuda.is_available() else "cpu"
    for key, val in DEVICE_PEAK_BF16.items():
        if key in name:
            return val
    return 1e12


def model_flops_per_token(cfg, seq_lens: Sequence[int] | None = None, backward: bool = True,
                          recompute: bool = False) -> float:
    """Dense matmul FLOPs per token (2 * active params, x3 with backward, +1 forward if layers
    are recomputed) plus the causal attention term averaged over the given document lengths."""
    H, L = cfg.hidden_size, cfg.num_hidden_layers
    attn_proj = H * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * H
    per_layer = 0.0
    for i in range(L):
        if cfg.layer_is_moe(i):
            mlp = 3 * H * cfg.moe_intermediate_size * cfg.num_experts_per_tok + H * cfg.num_experts \
                + 3 * H * cfg.shared_expert_intermediate_size
        else:
            mlp = 3 * H * cfg.intermediate_size
        per_layer += attn_proj + mlp
    active = per_layer + cfg.vocab_size * H
    mult = (3.0 if backward else 1.0) + (1.0 if (recompute and backward) else 0.0)
    flops = 2.0 * active * mult
    if seq_lens:
        tot = float(sum(seq_lens))
        sq = float(sum(l * l for l in seq_lens))
        # causal: QK^T and PV each 2*l*l*D/2 per head per document -> per token average
        attn_fwd = 2.0 * 2.0 * (sq / 2.0) * cfg.head_dim * cfg.num_attention_heads * L / max(tot, 1.0)
        flops += attn_fwd * ((3.5 if backward else 1.0) + (1.0 if (recompute and backward) else 0.0))
    return flops
