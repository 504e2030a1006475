"""Mixture-of-experts block: router, stacked experts, load-balancing loss, expert parallelism.

Parameter layout matches the reference (src/xorl/models/layers/moe/experts.py:1576-1584):
``mlp.gate.weight [E, H]``, ``mlp.experts.gate_up_proj [E, H, 2I]``, ``mlp.experts.down_proj
[E, I, H]``.  Routing is softmax -> top-k -> optional renormalisation in fp32
(src/xorl/models/layers/moe/router.py:232-259); the auxiliary loss is the switch-style
load-balancing loss ``E * sum_e f_e * P_e`` (src/xorl/models/layers/moe/aux_loss.py:67).
With expert parallelism the expert tensors hold only the local ``E / ep`` experts and tokens are
exchanged through ``xorl_b200.parallel.ep`` (all-to-all baseline or the fused peer-memory path).
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from ..ops import moe as moe_ops
from ..parallel.state import get_parallel_state
from .config import ModelConfig
from .context import StepContext
from .layers import MLP, Linear


class _RouterLogits(torch.autograd.Function):
    """fp32 logits = x @ W^T from bf16 operands (one GEMM launch); the backward GEMMs take the
    logit gradient rounded to bf16."""

    @staticmethod
    def forward(ctx, x, w):
        from ..ops.gemm import gemm
        ctx.save_for_backward(x)
        ctx.w = w
        return gemm(x, w, out_dtype=torch.float32)

    @staticmethod
    def backward(ctx, dl):
        from ..ops.gemm import gemm, weight_grad
        (x,) = ctx.saved_tensors
        w = ctx.w
        d = dl.to(torch.bfloat16)
        dx = gemm(d, w, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = weight_grad(d, x, w) if ctx.needs_input_grad[1] else None
        return dx, dw


def router_logits(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _RouterLogits.apply(x, w)


class TopKRouter(nn.Module):
    def __init__(self, cfg: ModelConfig, dtype=None, device=None):
        super().__init__()
        self.top_k = cfg.num_experts_per_tok
        self.num_experts = cfg.num_experts
        self.norm_topk_prob = cfg.norm_topk_prob
        self.scoring = cfg.scoring_func
        self.scale = cfg.routed_scaling_factor
        self.weight = nn.Parameter(torch.empty(cfg.num_experts, cfg.hidden_size, dtype=dtype, device=device))
        self.bias = nn.Parameter(torch.zeros(cfg.num_experts, dtype=dtype, device=device)) \
            if cfg.router_bias else None
        self.n_group, self.topk_group = cfg.n_group, cfg.topk_group
        # selection-only bias of auxiliary-loss-free balancing: not trained by gradient descent
        self.e_score_correction_bias = nn.Parameter(
            torch.zeros(cfg.num_experts, dtype=torch.float32, device=device), requires_grad=False) \
            if cfg.extra.get("topk_method") == "noaux_tc" or cfg.extra.get("use_correction_bias") else None

    def forward(self, x: torch.Tensor):
        """x [T, H] -> (weights fp32 [T, k], indices int64 [T, k], probs fp32 [T, E])."""
        if x.is_cuda and x.dtype == torch.bfloat16 and self.weight.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0 \
                and self.weight.shape[0] % 8 == 0:
            # bf16 operands, fp32 accumulation and fp32 logits out of the tcgen05 GEMM: the same products
            # as an fp32 matmul of the bf16 values, without materialising fp32 copies of x and W
            logits = router_logits(x, self.weight)
            if self.bias is not None:
                logits = logits + self.bias.float()
        else:
            logits = torch.nn.functional.linear(x.float(), self.weight.float(),
                                                None if self.bias is None else self.bias.float())
        return moe_ops.topk_route(logits, self.top_k, self.norm_topk_prob, self.scoring, self.scale,
                                  self.n_group, self.topk_group, self.e_score_correction_bias)


class Experts(nn.Module):
    """Stacked expert weights; ``num_local`` experts live on this rank."""

    def __init__(self, cfg: ModelConfig, num_local: int, dtype=None, device=None, hidden: Optional[int] = None,
                 gated: bool = True, activation: Optional[str] = None):
        """``hidden``: width the experts work on (a latent width for Nemotron-H); ``gated=False``
        with ``activation="relu2"``: ``down(relu(up(x))^2)``, the up projection stored in
        ``gate_up_proj [E, H, I]``."""
        super().__init__()
        H, I = hidden or cfg.hidden_size, cfg.moe_intermediate_size
        self.num_local = num_local
        self.activation = activation
        # block-scaled fp8 expert GEMMs (train.enable_fp8_training): None, "fp8" or "bf16" = precision
        # of the input-gradient GEMM (train.fp8_training_backward)
        self.fp8_mode: Optional[str] = None
        self.gate_up_proj = nn.Parameter(torch.empty(num_local, H, (2 if gated else 1) * I, dtype=dtype, device=device))
        self.down_proj = nn.Parameter(torch.empty(num_local, I, H, dtype=dtype, device=device))
        self.gate_up_proj._xb_expert = True
        self.down_proj._xb_expert = True
        self.swiglu_limit = cfg.swiglu_limit
        self.gate_up_bias = self.down_bias = None
        if cfg.expert_bias:
            self.gate_up_bias = nn.Parameter(torch.zeros(num_local, 2 * I, dtype=dtype, device=device))
            self.down_bias = nn.Parameter(torch.zeros(num_local, H, dtype=dtype, device=device))
            self.gate_up_bias._xb_expert = True
            self.down_bias._xb_expert = True
        ps = get_parallel_state()
        if ps.ep_size > 1 and num_local * ps.ep_size == cfg.num_experts:
            from ..parallel.ep import mark_ep
            for prm in (self.gate_up_proj, self.down_proj, self.gate_up_bias, self.down_bias):
                if prm is not None:
                    mark_ep(prm, ps.rank_in("ep"), ps.ep_size)

    def mlp_kwargs(self):
        kw = {}
        if not (self.gate_up_bias is None and self.swiglu_limit is None and self.activation is None):
            kw = dict(gate_up_bias=self.gate_up_bias, down_bias=self.down_bias, swiglu_limit=self.swiglu_limit)
            if self.activation is not None:
                kw["activation"] = self.activation
        if self.fp8_mode is not None:
            kw["fp8"] = self.fp8_mode
        lora = getattr(self, "lora", None)
        if lora is not None and lora.tensors() is not None:
            kw["lora"] = lora.tensors()
        return kw

    def forward(self, x_sorted: torch.Tensor, tokens_per_expert: torch.Tensor) -> torch.Tensor:
        """x_sorted [M, H] grouped by local expert; tokens_per_expert int64 [num_local]."""
        return moe_ops.expert_mlp(x_sorted, tokens_per_expert, self.gate_up_proj, self.down_proj,
                                  **self.mlp_kwargs())


class MoEBlock(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.cfg = cfg
        self.layer_idx = layer_idx
        ps = get_parallel_state()
        self.ep_size = ps.ep_size
        if cfg.num_experts % self.ep_size:
            raise ValueError(f"num_experts {cfg.num_experts} not divisible by ep {self.ep_size}")
        self.num_local = cfg.num_experts // self.ep_size
        self.gate = TopKRouter(cfg, dtype=dtype, device=device)
        self.experts = self.build_experts(cfg, dtype, device)
        self.shared_expert = None
        if cfg.shared_expert_intermediate_size:
            self.shared_expert = MLP(cfg.hidden_size, cfg.shared_expert_intermediate_size,
                                     dtype=dtype, device=device, swiglu_limit=cfg.extra.get("dense_swiglu_limit"))
        # Qwen3-Next / Qwen3.5 MoE: the shared expert is scaled by sigmoid(w_g . x) per token
        self.shared_expert_gate = Linear(cfg.hidden_size, 1, dtype=dtype, device=device) \
            if (self.shared_expert is not None and cfg.extra.get("shared_expert_gate")) else None
        self.aux_coef = cfg.router_aux_loss_coef
        # gradient of the expert outputs with respect to the routing weights reaches the router only
        # when this is set (``model.train_router``; src/xorl/arguments.py:491-497)
        self.train_router = True
        self.moe_ordinal = sum(cfg.layer_is_moe(i) for i in range(layer_idx))

    def build_experts(self, cfg: ModelConfig, dtype, device) -> "Experts":
        return Experts(cfg, self.num_local, dtype=dtype, device=device)

    def pre_experts(self, x: torch.Tensor) -> torch.Tensor:
        """Hook: what the routed experts see (identity; a latent projection for Nemotron-H)."""
        return x

    def post_experts(self, y: torch.Tensor) -> torch.Tensor:
        return y

    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        T, H = x.shape
        replay = ctx.aux.get(("routing_replay", self.layer_idx))
        weights, indices, probs = self.gate(x)
        allr = ctx.aux.get("routing_replay_all")
        if replay is None and allr is not None:
            # rollout routing replay: [T, moe_layers, k]; rows of -1 keep the router's own choice
            r = allr[:, self.moe_ordinal]
            replay = torch.where(r >= 0, r, indices)
        if replay is not None:
            # replay recorded expert choices (recompute / pipeline backward / rollout routing);
            # the weights are re-derived from the current probabilities so gradients still flow
            indices = replay
            weights = probs.gather(1, indices)
            if self.cfg.norm_topk_prob:
                weights = weights / weights.sum(-1, keepdim=True).clamp_min(1e-20)
            if self.gate.scale != 1.0 and self.gate.scoring != "softmax_after_topk":
                weights = weights * self.gate.scale
        elif ctx.aux.get("record_routing", False):
            ctx.aux[("routing_record", self.layer_idx)] = indices.detach()
        counts = None
        if ctx.training and self.aux_coef > 0 and ctx.aux.get("aux_loss_scale") is not None:
            counts = moe_ops.expert_histogram(indices, self.cfg.num_experts)
            aux = moe_ops.load_balancing_loss(probs, indices, self.cfg.num_experts,
                                              ctx.aux.get("aux_global_group"), counts=counts)
            ctx.aux[("aux_loss", self.layer_idx)] = aux * (self.aux_coef * ctx.aux["aux_loss_scale"])
        if ctx.aux.get("collect_expert_load", False):
            if counts is None:
                counts = moe_ops.expert_histogram(indices, self.cfg.num_experts)
            ctx.aux[("expert_load", self.layer_idx)] = counts.long()
        if not self.train_router:
            weights = weights.detach()
        xe = self.pre_experts(x)
        if self.ep_size > 1:
            from ..parallel import ep as ep_ops
            out = ep_ops.ep_moe_forward(xe, weights, indices, self.experts, self.cfg.num_experts, ctx)
        else:
            out = moe_ops.local_moe_forward(xe, weights, indices, self.experts, self.cfg.num_experts,
                                            canonical=bool(ctx.aux.get("canonical_moe", False)))
        out = self.post_experts(out)
        if self.shared_expert is not None:
            sh = self.shared_expert(x)
            if self.shared_expert_gate is not None:
                sh = sh * torch.sigmoid(torch.nn.functional.linear(x.float(), self.shared_expert_gate.weight.float())).to(sh.dtype)
            out = out + sh
        return out
