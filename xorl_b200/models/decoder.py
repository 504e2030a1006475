"""Generic decoder-only language model used by the dense and MoE families.

The model is organised as *units* — embedding, each decoder layer, head (final norm + lm_head) —
which is the granularity at which the ZeRO-3 engine gathers parameters, recomputes activations
and reduce-scatters gradients.  Between units the activation is the pair ``(h, residual)`` whose
sum is the residual stream, so every RMSNorm runs fused with the preceding residual add
(src/xorl/models/transformers/qwen3/modeling_qwen3.py:98-156 has the same fused pre-norm).
Without an engine, ``forward`` runs everything under ordinary autograd.
"""
from __future__ import annotations

from typing import Any, Dict, Optional

import torch
from torch import nn

from ..ops import embedding as emb_ops
from ..ops import loss as loss_ops
from .config import ModelConfig
from .context import StepContext, cu_seqlens_from_position_ids, packed_metadata_from_padded
from .layers import MLP, Attention, Linear, RMSNorm
from .rope import RotaryEmbedding


def _sequence_parallel() -> bool:
    from ..parallel.state import get_parallel_state
    return bool(get_parallel_state().tp_sequence_parallel)


class DecoderLayer(nn.Module):
    def __init__(self, cfg: ModelConfig, layer_idx: int, dtype=None, device=None):
        super().__init__()
        self.layer_idx = layer_idx
        self.post_norm = cfg.norm_placement == "post"
        if cfg.layer_types is not None and cfg.layer_types[layer_idx] == "linear_attention":
            from .gated_deltanet import GatedDeltaNet
            self.self_attn = GatedDeltaNet(cfg, layer_idx, dtype=dtype, device=device)
        elif cfg.model_type == "glm5":
            from .glm5 import Glm5Attention
            self.self_attn = Glm5Attention(cfg, layer_idx, dtype=dtype, device=device)
        elif cfg.extra.get("kv_lora_rank"):
            from .mla import MLAttention
            self.self_attn = MLAttention(cfg, layer_idx, dtype=dtype, device=device)
        elif cfg.model_type == "minimax_m3":
            from .minimax_m3 import MiniMaxAttention
            self.self_attn = MiniMaxAttention(cfg, layer_idx, dtype=dtype, device=device)
        else:
            self.self_attn = Attention(cfg, layer_idx, dtype=dtype, device=device)
        if cfg.layer_is_moe(layer_idx):
            from .moe import MoEBlock
            self.mlp = MoEBlock(cfg, layer_idx, dtype=dtype, device=device)
        else:
            self.mlp = MLP(cfg.hidden_size, cfg.intermediate_size, cfg.mlp_bias, dtype=dtype,
                           device=device, swiglu_limit=cfg.extra.get("dense_swiglu_limit"))
        zc = cfg.zero_centered_norm
        if self.post_norm:
            self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, zc, dtype, device)
            self.post_feedforward_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, zc, dtype, device)
        else:
            self.input_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, zc, dtype, device)
            self.post_attention_layernorm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, zc, dtype, device)
        if _sequence_parallel():
            # every tensor-parallel rank normalises its own tokens: replicated weights that act on
            # token shards get partial gradients, summed over the group before the optimizer step
            if not (isinstance(self.self_attn, Attention) and isinstance(self.mlp, MLP)):
                raise NotImplementedError("tensor_parallel_sequence_parallel supports dense attention + MLP layers")
            for n, p in self.named_parameters():
                if "layernorm" in n or n == "mlp.down_proj.bias":
                    p._xb_tp_reduce = True

    def forward(self, h: torch.Tensor, residual: Optional[torch.Tensor], ctx: StepContext):
        if self.post_norm:
            x = h if residual is None else h + residual
            x = x + self.post_attention_layernorm(self.self_attn(x, ctx))
            x = x + self.post_feedforward_layernorm(self._mlp(x, ctx))
            return x, None
        if residual is None:
            y, x = self.input_layernorm(h), h
        else:
            y, x = self.input_layernorm(h, residual=residual)
        a = self.self_attn(y, ctx)
        y, x = self.post_attention_layernorm(a, residual=x)
        return self._mlp(y, ctx), x

    def _mlp(self, y, ctx):
        if isinstance(self.mlp, MLP):
            return self.mlp(y)
        return self.mlp(y, ctx)


class DecoderLM(nn.Module):
    """Causal language model over packed sequences."""

    def __init__(self, cfg: ModelConfig, dtype=None, device=None, layer_indices=None,
                 has_embed: bool = True, has_head: bool = True):
        """``layer_indices`` / ``has_embed`` / ``has_head`` build only a pipeline stage's part of
        the model; layers keep their global index in their name (``layers.{i}``)."""
        super().__init__()
        self.config = cfg
        self.has_embed, self.has_head = has_embed, has_head
        idx = list(range(cfg.num_hidden_layers)) if layer_indices is None else list(layer_indices)
        self.layer_indices = idx
        if has_embed:
            self.embed_tokens = nn.Embedding(cfg.vocab_size, cfg.hidden_size, dtype=dtype, device=device)
        layer_cls = DecoderLayer
        if cfg.model_type == "nemotron_h":
            from .nemotron_h import NemotronHLayer
            layer_cls = NemotronHLayer
        elif cfg.model_type == "deepseek_v4":
            from .deepseek_v4 import HyperConnection, V4Layer
            layer_cls = V4Layer
            if has_head:
                self.hc_head = HyperConnection(cfg, device=device, head=True)
        self.layers = nn.ModuleDict({str(i): layer_cls(cfg, i, dtype, device) for i in idx})
        if has_head:
            self.norm = RMSNorm(cfg.hidden_size, cfg.rms_norm_eps, cfg.zero_centered_norm, dtype, device)
            from ..parallel.tp import tp_info
            tp, tp_rank, tp_group = tp_info()
            # untied heads are sharded by vocabulary rows over the tensor-parallel group and use
            # the vocab-parallel loss; tied heads stay replicated with the embedding
            self.vocab_parallel = tp > 1 and not cfg.tie_word_embeddings and cfg.vocab_size % tp == 0
            self.head_tp = (tp, tp_rank, tp_group)
            # lm-head-only tensor parallelism (train.lm_head_tensor_parallel_size): the body is data parallel,
            # only the head is split by vocabulary rows over groups of consecutive data-parallel ranks, which
            # pool their tokens for the loss (src/xorl/distributed/parallel_state.py:64-116,781-830)
            from ..parallel.state import get_parallel_state
            ps = get_parallel_state()
            lm_tp = getattr(ps, "lm_head_tp_size", 1)
            self.head_gathers_tokens = False
            if tp == 1 and lm_tp > 1:
                if cfg.tie_word_embeddings or cfg.vocab_size % lm_tp:
                    raise ValueError("lm_head_tensor_parallel_size needs an untied lm-head whose vocabulary divides by it")
                self.vocab_parallel, self.head_gathers_tokens = True, True
                self.head_tp = (lm_tp, ps.rank_in("lm_head_tp"), ps.group("lm_head_tp"))
            v_local = cfg.vocab_size // self.head_tp[0] if self.vocab_parallel else cfg.vocab_size
            self.lm_head = Linear(cfg.hidden_size, v_local, bias=False, dtype=dtype, device=device)
            if self.head_gathers_tokens:
                from ..parallel.tp import mark_lm_head
                mark_lm_head(self.lm_head.weight, (cfg.vocab_size, cfg.hidden_size), self.head_tp[0], self.head_tp[1])
            elif self.vocab_parallel:
                from ..parallel.tp import mark_col
                mark_col(self.lm_head.weight, (cfg.vocab_size, cfg.hidden_size), (cfg.vocab_size,))
        if cfg.tie_word_embeddings and has_embed and has_head:
            self.lm_head.weight = self.embed_tokens.weight
        elif cfg.tie_word_embeddings and (has_embed != has_head):
            raise ValueError("tied embeddings cannot be split across pipeline stages")
        self.rotary = RotaryEmbedding(cfg.head_dim, cfg.rope_theta, cfg.rope_scaling,
                                      cfg.partial_rotary_factor, cfg.max_position_embeddings)
        self.sp = None
        if _sequence_parallel():
            from ..parallel.tp_fused import sp_context
            self.sp = sp_context()
            if cfg.tie_word_embeddings:
                raise NotImplementedError("tensor_parallel_sequence_parallel needs untied embeddings")
            if has_embed:
                self.embed_tokens.weight._xb_tp_reduce = True     # each rank embeds its own tokens
            if has_head:
                self.norm.weight._xb_tp_reduce = True
        self.loss_chunk_tokens = 1024
        self.cp_strategy = None
        self.ctx_defaults = {}          # copied into every StepContext.aux (ep_dispatch, ...)
        self.aux_loss_enabled = False   # MoE load-balancing loss (set by the trainer)

    # ---- initialisation ---------------------------------------------------------------------
    @torch.no_grad()
    def init_weights(self, seed: int = 0) -> None:
        """N(0, initializer_range) for matrices and embeddings, ones (zeros if zero-centred) for
        norm weights, zeros for biases.  Each parameter draws from its own generator seeded by
        (seed, position in named_parameters) so the result does not depend on how parameters are
        later sharded."""
        std = self.config.initializer_range
        for idx, (name, p) in enumerate(self.named_parameters()):
            init_parameter_(name, p, std, seed, idx, self.config.zero_centered_norm, self.config.num_experts)

    # ---- unit-level API used by the engine ------------------------------------------------------
    def make_context(self, input_ids, position_ids=None, cu_seqlens=None, causal=True,
                     training=True, extra=None) -> StepContext:
        dev = input_ids.device
        if input_ids.dim() == 2 and position_ids is None and cu_seqlens is None:
            B, S = input_ids.shape
            cu_seqlens, position_ids = packed_metadata_from_padded(B, S, dev)
        if position_ids is None:
            cu = cu_seqlens.to(torch.int64)
            T = input_ids.numel()
            idx = torch.arange(T, device=dev)
            seg = torch.searchsorted(cu[1:].contiguous(), idx, right=True)
            position_ids = idx - cu[seg]
        position_ids = position_ids.reshape(-1)
        if cu_seqlens is None:
            cu_seqlens = cu_seqlens_from_position_ids(position_ids)
        cu_seqlens = cu_seqlens.to(device=dev, dtype=torch.int32)
        ctx = StepContext(cu_seqlens=cu_seqlens, position_ids=position_ids, causal=causal,
                          training=training, cp=self.cp_strategy)
        ctx.aux.update(self.ctx_defaults)
        if self.config.extra.get("num_hash_layers"):
            ctx.aux["input_ids"] = input_ids.reshape(-1)       # hash-routed MoE layers pick experts by token id
        if extra:
            ctx.aux.update({k: v for k, v in extra.items() if v is not None})
        if ctx.cp is not None:
            ctx.cp.prepare(self, ctx)
        else:
            ctx.cos, ctx.sin = self.rotary(position_ids)
        return ctx

    def forward_embed(self, input_ids: torch.Tensor, ctx: StepContext):
        ids = input_ids.reshape(-1)
        if self.config.model_type == "deepseek_v4":
            # hyper-connections: the residual stream starts as hc_mult copies of the embedding
            e = emb_ops.embedding(ids, self.embed_tokens.weight)
            return e.unsqueeze(1).repeat(1, int(self.config.extra.get("hc_mult", 4)), 1), None
        if self.sp is not None:
            from ..parallel.tp_fused import local_tokens
            ids = local_tokens(ids, self.sp)        # the residual stream holds T / tp tokens per rank
        return emb_ops.embedding(ids, self.embed_tokens.weight), None

    def forward_head(self, h, residual, ctx: StepContext) -> torch.Tensor:
        if self.config.model_type == "deepseek_v4":
            return self.norm(self.hc_head.collapse(h))
        hidden = self.norm(h) if residual is None else self.norm(h, residual=residual)[0]
        if self.sp is not None:
            # the loss sees all tokens on every rank and returns the same gradient everywhere
            from ..parallel.tp_fused import gather_tokens
            hidden = gather_tokens(hidden, self.sp)
        return hidden

    def head_loss(self, h, residual, labels: torch.Tensor, ctx: StepContext, grad_scale: float = 1.0,
                  return_token_losses: bool = False):
        """grad_scale * sum of token cross-entropies (labels == -100 ignored)."""
        hidden = self.forward_head(h, residual, ctx)
        distill = ctx.aux.get("distill")
        if distill is not None:
            # teacher-student KL on the same hidden states, added to the cross-entropy with the same
            # token normalisation (``distill.distillation_loss_weight``)
            t_hidden, t_weight, kind, weight = distill
            from ..ops import kl_losses
            if getattr(self, "head_gathers_tokens", False):
                raise NotImplementedError("distillation is not supported with lm_head_tensor_parallel_size > 1")
            if getattr(self, "vocab_parallel", False):
                # both lm-heads are row-sharded over the tensor-parallel group: the divergence is formed
                # from local logit shards, only per-token statistics cross the group
                tp, tp_rank, tp_group = self.head_tp
                kl = kl_losses.vocab_parallel_kl(hidden, self.lm_head.weight, t_hidden, t_weight, labels,
                                                 tp_group, kind).sum()
                loss = loss_ops.vocab_parallel_linear_cross_entropy(
                    hidden, self.lm_head.weight, labels.reshape(-1), tp_group,
                    tp_rank * (self.config.vocab_size // tp), grad_scale, self.loss_chunk_tokens)
                ctx.aux["distill_kl"] = kl.detach() * grad_scale
                total = loss + kl * (weight * grad_scale)
                return (total, None) if return_token_losses else total
            # exact full-vocabulary divergence streamed over vocabulary chunks: [tokens, chunk] peak memory
            kl = kl_losses.streaming_kl(hidden, self.lm_head.weight, t_hidden, t_weight, labels, kind,
                                        vocab_chunk=int(getattr(self, "distill_vocab_chunk", 16384))).sum()
            ce = loss_ops.fused_linear_cross_entropy(hidden, self.lm_head.weight, labels.reshape(-1), grad_scale,
                                                     self.loss_chunk_tokens,
                                                     z_loss=float(getattr(self, "z_loss_coef", 0.0)))
            ctx.aux["distill_kl"] = kl.detach() * grad_scale
            total = ce + kl * (weight * grad_scale)
            return (total, None) if return_token_losses else total
        if getattr(self, "vocab_parallel", False):
            if getattr(self, "z_loss_coef", 0.0):
                raise NotImplementedError("softmax_auxiliary_loss (z-loss) is not supported with a "
                                          "vocabulary-parallel lm-head")
            tp, tp_rank, tp_group = self.head_tp
            pooled = getattr(self, "head_gathers_tokens", False)
            # pooled: every rank of the lm-head group brings its own tokens; the loss streams the group's
            # tokens chunk by chunk through this rank's vocabulary rows and returns the group total
            loss = loss_ops.vocab_parallel_linear_cross_entropy(
                hidden, self.lm_head.weight, labels.reshape(-1), tp_group,
                tp_rank * (self.config.vocab_size // tp), grad_scale, self.loss_chunk_tokens, pooled=pooled)
            if pooled:
                from ..parallel.tp import _OwnShare
                loss = _OwnShare.apply(loss, tp)        # this rank's share: the shares add up to the total
            return (loss, None) if return_token_losses else loss
        return loss_ops.fused_linear_cross_entropy(hidden, self.lm_head.weight, labels.reshape(-1),
                                                   grad_scale, self.loss_chunk_tokens,
                                                   z_loss=float(getattr(self, "z_loss_coef", 0.0)),
                                                   return_token_losses=return_token_losses)

    def unit_modules(self):
        """(name, modules) per ZeRO unit, in execution order.  The root unit (embedding, final
        norm, lm_head) stays gathered for the whole step."""
        root = []
        if self.has_embed:
            root.append(self.embed_tokens)
        if self.has_head:
            root += [self.norm, self.lm_head]
            if hasattr(self, "hc_head"):
                root.append(self.hc_head)
        units = [("root", root)] if root else []
        return units + [(f"layers.{i}", [l]) for i, l in self.layers.items()]

    # ---- plain autograd forward --------------------------------------------------------------
    def forward(self, input_ids, labels=None, position_ids=None, cu_seqlens=None,
                grad_scale: float = 1.0, return_hidden: bool = False) -> Dict[str, Any]:
        ctx = self.make_context(input_ids, position_ids, cu_seqlens, training=self.training)
        h, res = self.forward_embed(input_ids, ctx)
        for layer in self.layers.values():
            h, res = layer(h, res, ctx)
        out: Dict[str, Any] = {"aux": ctx.aux}
        if labels is not None:
            out["loss"] = self.head_loss(h, res, labels, ctx, grad_scale)
        if return_hidden or labels is None:
            out["last_hidden_state"] = self.forward_head(h, res, ctx)
        return out

    @torch.no_grad()
    def logits(self, input_ids, position_ids=None, cu_seqlens=None) -> torch.Tensor:
        hid = self.forward(input_ids, None, position_ids, cu_seqlens)["last_hidden_state"]
        return torch.nn.functional.linear(hid, self.lm_head.weight)


@torch.no_grad()
def init_parameter_(name: str, p: torch.Tensor, std: float, seed: int, index: int,
                    zero_centered_norm: bool = False, num_experts: int = 0) -> None:
    if p.is_meta:
        return
    if ".lora_A." in name or ".lora_B." in name or name.endswith("_lora_A") or name.endswith("_lora_B"):
        from ..adapters.lora import init_lora_parameter_
        init_lora_parameter_(name, p, 0, seed)
        return
    leaf = name.rsplit(".", 1)[-1]
    if ".mixer." in name and leaf in ("A_log", "D", "dt_bias", "norm_weight", "conv1d_bias"):
        import zlib
        from .mamba2 import init_mamba_parameter_
        g = torch.Generator(device="cpu").manual_seed((seed * 1000003 + zlib.crc32(name.encode()) * 7919 + 17) % (2 ** 63 - 1))
        tmp = torch.empty(p.shape, dtype=torch.float32)
        init_mamba_parameter_(name, tmp, g)
        p.copy_(tmp.to(p.device))
        return
    if leaf in ("attn_sink", "base") or leaf == "tid2eid":
        if leaf == "tid2eid":
            import zlib
            from .deepseek_v4 import init_hash_table_
            g = torch.Generator(device="cpu").manual_seed((seed * 1000003 + zlib.crc32(name.encode()) * 7919 + 17) % (2 ** 63 - 1))
            tmp = torch.empty(p.shape, dtype=torch.float32)
            init_hash_table_(tmp, num_experts or p.shape[1], g)
            p.copy_(tmp.to(p.device))
        else:
            p.zero_()
        return
    if leaf == "A_log":                      # GatedDeltaNet decay rates spread over (0, 16)
        p.copy_(torch.linspace(0.5, 16.0, p.numel()).log().to(p.device))
        return
    if leaf in ("dt_bias", "o_norm_weight"):  # unit step bias / plain (not zero-centred) gated norm
        p.fill_(1.0)
        return
    if leaf == "sinks":
        p.zero_()
        return
    if p.dim() == 1:
        if leaf == "bias" or "bias" in leaf:
            p.zero_()
        elif zero_centered_norm:
            p.zero_()
        else:
            p.fill_(1.0)
        return
    import zlib
    # seeded by the parameter *name*, so a pipeline stage that builds only some layers draws the
    # same values for them as a process that builds the whole model
    index = zlib.crc32(name.encode())
    g = torch.Generator(device="cpu").manual_seed((seed * 1000003 + index * 7919 + 17) % (2 ** 63 - 1))
    if p.numel() <= (1 << 24) or p.device.type == "cpu":
        vals = torch.empty(p.shape, dtype=torch.float32).normal_(0.0, std, generator=g)
        p.copy_(vals.to(p.device))
    else:
        # large tensors: draw on the device (still deterministic per (seed, index))
        gd = torch.Generator(device=p.device).manual_seed((seed * 1000003 + index * 7919 + 17) % (2 ** 63 - 1))
        p.copy_(torch.empty(p.shape, dtype=torch.float32, device=p.device).normal_(0.0, std, generator=gd))
