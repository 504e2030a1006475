"""Model configuration shared by every decoder family.

Reads Hugging Face ``config.json`` files (or a plain dict) and normalises the family-specific
spellings into one dataclass; the per-family registry entries in ``registry.py`` only set flags.
Covers the fields the reference's family configs read (src/xorl/models/transformers/*/configuration_*.py).
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass, field, fields
from typing import Any, Dict, List, Optional


@dataclass
class ModelConfig:
    model_type: str = "qwen3"
    architectures: List[str] = field(default_factory=list)
    vocab_size: int = 151936
    hidden_size: int = 4096
    intermediate_size: int = 12288
    num_hidden_layers: int = 36
    num_attention_heads: int = 32
    num_key_value_heads: int = 8
    head_dim: Optional[int] = None
    hidden_act: str = "silu"
    max_position_embeddings: int = 40960
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    rope_scaling: Optional[Dict[str, Any]] = None
    partial_rotary_factor: float = 1.0
    tie_word_embeddings: bool = False
    attention_bias: bool = False
    attention_dropout: float = 0.0
    mlp_bias: bool = False
    use_qk_norm: bool = True
    qk_norm_full: bool = False          # olmo2: RMSNorm over the whole projection, not per head
    norm_placement: str = "pre"         # "pre" (llama/qwen) or "post" (olmo2)
    zero_centered_norm: bool = False
    sliding_window: Optional[int] = None
    layer_types: Optional[List[str]] = None
    initializer_range: float = 0.02
    torch_dtype: str = "bfloat16"
    # ---- mixture of experts -----------------------------------------------------------------
    num_experts: int = 0
    num_experts_per_tok: int = 0
    moe_intermediate_size: int = 0
    shared_expert_intermediate_size: int = 0
    n_shared_experts: int = 0
    norm_topk_prob: bool = True
    decoder_sparse_step: int = 1
    mlp_only_layers: List[int] = field(default_factory=list)
    first_k_dense_replace: int = 0
    router_aux_loss_coef: float = 0.001
    output_router_logits: bool = False
    scoring_func: str = "softmax"       # softmax | sigmoid
    routed_scaling_factor: float = 1.0
    n_group: int = 1
    topk_group: int = 1
    router_bias: bool = False
    expert_bias: bool = False
    swiglu_limit: Optional[float] = None
    attention_sinks: bool = False
    extra: Dict[str, Any] = field(default_factory=dict)

    def __post_init__(self):
        if self.head_dim is None:
            self.head_dim = self.hidden_size // self.num_attention_heads
        if self.num_key_value_heads is None:
            self.num_key_value_heads = self.num_attention_heads

    # -- derived ------------------------------------------------------------------------------
    @property
    def is_moe(self) -> bool:
        return self.num_experts > 0

    def layer_is_moe(self, idx: int) -> bool:
        if self.extra.get("layers_block_type"):
            return self.extra["layers_block_type"][idx] == "moe"
        if not self.is_moe or idx in self.mlp_only_layers or idx < self.first_k_dense_replace:
            return False
        return (idx + 1) % max(1, self.decoder_sparse_step) == 0

    @property
    def q_size(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_size(self) -> int:
        return self.num_key_value_heads * self.head_dim

    def num_parameters(self, include_embeddings: bool = True) -> int:
        H, I, L = self.hidden_size, self.intermediate_size, self.num_hidden_layers
        attn = H * (self.q_size + 2 * self.kv_size) + self.q_size * H
        if self.use_qk_norm:
            attn += 2 * self.head_dim
        total = 0
        for i in range(L):
            total += attn + 2 * H
            if self.layer_is_moe(i):
                total += H * self.num_experts + self.num_experts * 3 * H * self.moe_intermediate_size
                total += 3 * H * self.shared_expert_intermediate_size
            else:
                total += 3 * H * I
        total += H
        if include_embeddings:
            total += self.vocab_size * H * (1 if self.tie_word_embeddings else 2)
        return total

    # -- io -----------------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "ModelConfig":
        d = dict(d)
        known = {f.name for f in fields(cls)}
        # family-specific spellings
        if "num_local_experts" in d and "num_experts" not in d:
            d["num_experts"] = d.pop("num_local_experts")
        if "n_routed_experts" in d and "num_experts" not in d:
            d["num_experts"] = d.pop("n_routed_experts")
        if "experts_per_token" in d and "num_experts_per_tok" not in d:
            d["num_experts_per_tok"] = d.pop("experts_per_token")
        if "rope_parameters" in d and isinstance(d["rope_parameters"], dict):
            rp = d.pop("rope_parameters")
            d.setdefault("rope_theta", rp.get("rope_theta", 1e6))
            if rp.get("rope_type", "default") != "default":
                d.setdefault("rope_scaling", rp)
        mt = d.get("model_type", "qwen3")
        if "use_qk_norm" not in d:
            d["use_qk_norm"] = mt in ("qwen3", "qwen3_moe", "olmo2", "qwen3_5", "qwen3_5_moe", "glm4_moe",
                                      "minimax_m3", "minimax_m3_vl", "xorl_minimax_m3") and d.get("use_qk_norm", True)
        if mt == "olmo2":
            d.setdefault("norm_placement", "post")
            d.setdefault("qk_norm_full", True)
        if mt in ("qwen2",):
            d.setdefault("attention_bias", True)
            d["use_qk_norm"] = False
        if mt in ("llama",):
            d["use_qk_norm"] = False
        if mt in ("qwen3_5", "qwen3_5_moe", "qwen3_next"):
            d["use_qk_norm"] = True
            d.setdefault("zero_centered_norm", True)
            d.setdefault("partial_rotary_factor", 0.25)
            d.setdefault("attn_output_gate", True)
            if d.get("layer_types") is None:
                n, every = d.get("num_hidden_layers", 0), d.get("full_attention_interval", 4)
                d["layer_types"] = ["full_attention" if (i + 1) % every == 0 else "linear_attention" for i in range(n)]
            if mt == "qwen3_5_moe" or d.get("num_experts"):
                d.setdefault("shared_expert_gate", bool(d.get("shared_expert_intermediate_size")))
        if mt == "gpt_oss":
            d["use_qk_norm"] = False
            d.setdefault("attention_bias", True)
            d.setdefault("attention_sinks", True)
            d.setdefault("expert_bias", True)
            d.setdefault("router_bias", True)
            d.setdefault("swiglu_limit", 7.0)
            d.setdefault("scoring_func", "softmax_after_topk")
            d.setdefault("norm_topk_prob", False)
            d.setdefault("moe_intermediate_size", d.get("intermediate_size", 0))
            if d.get("layer_types") is None and d.get("sliding_window"):
                n = d.get("num_hidden_layers", 0)
                d["layer_types"] = ["sliding_attention" if i % 2 == 0 else "full_attention" for i in range(n)]
        if mt in ("glm5", "glm_moe_dsa", "xorl_glm5"):
            if isinstance(d.get("text_config"), dict):
                d = {**{k: v for k, v in d.items() if k != "text_config"}, **d["text_config"]}
            mt = d["model_type"] = "glm5"
            d.setdefault("topk_method", "noaux_tc")
        if mt in ("deepseek_v3", "glm4_moe", "glm5"):
            d["use_qk_norm"] = bool(d.get("use_qk_norm", False)) if mt == "glm4_moe" else False
            d.setdefault("scoring_func", "sigmoid")
            d.setdefault("use_correction_bias", True)
            if d.get("n_shared_experts") and not d.get("shared_expert_intermediate_size"):
                d["shared_expert_intermediate_size"] = d["n_shared_experts"] * d.get("moe_intermediate_size", 0)
            if mt == "deepseek_v3" and d.get("moe_layer_freq"):
                d.setdefault("decoder_sparse_step", d["moe_layer_freq"])
            if mt in ("deepseek_v3", "glm5"):
                d["head_dim"] = d.get("qk_rope_head_dim", 64)      # rotary table covers the rope slice
        if mt in ("minimax_m3", "minimax_m3_vl", "xorl_minimax_m3"):
            # the published config is a multimodal wrapper with the language model under text_config
            if isinstance(d.get("text_config"), dict):
                d = {**{k: v for k, v in d.items() if k not in ("text_config", "vision_config")}, **d["text_config"]}
            mt = d["model_type"] = "minimax_m3"
            d.pop("vision_config", None)
            d.setdefault("zero_centered_norm", bool(d.pop("use_gemma_norm", True)))
            d["use_qk_norm"] = bool(d.get("use_qk_norm", True))
            d.setdefault("qk_norm_per_head_weights", d.get("qk_norm_type", "per_head") == "per_head")
            hd = d.get("head_dim", 128)
            d.setdefault("partial_rotary_factor", d.get("rotary_dim", 64) / hd)
            d.setdefault("num_experts", d.get("num_local_experts", 128))
            d.pop("num_local_experts", None)
            d.setdefault("moe_intermediate_size", d.get("intermediate_size", 3072))
            d["intermediate_size"] = d.get("dense_intermediate_size", 12288)
            d.setdefault("shared_expert_intermediate_size",
                         d.get("shared_intermediate_size", 3072) * d.get("n_shared_experts", 1))
            d.setdefault("scoring_func", "sigmoid")
            d.setdefault("use_correction_bias", bool(d.get("use_routing_bias", True)))
            d.setdefault("routed_scaling_factor", 2.0)
            d.setdefault("norm_topk_prob", True)
            d.setdefault("swiglu_limit", 7.0)
            d.setdefault("dense_swiglu_limit", d["swiglu_limit"])
            d.setdefault("router_aux_loss_coef", 0.0)
            n = d.get("num_hidden_layers", 60)
            freq = d.get("moe_layer_freq")
            if freq is not None:
                d.setdefault("mlp_only_layers", [i for i, f in enumerate(freq) if not f])
            sa = d.pop("sparse_attention_config", None) or {}
            d.setdefault("sparse_attention_freq", list(sa.get("sparse_attention_freq") or [0] * n))
            for key, default in (("sparse_block_size", 128), ("sparse_topk_blocks", 16), ("sparse_num_index_heads", 4),
                                 ("sparse_index_dim", hd), ("sparse_init_block", 0), ("sparse_local_block", 1)):
                d.setdefault(key, sa.get(key, default))
        if mt == "deepseek_v4":
            d["use_qk_norm"] = False
            d["v4_head_dim"] = d.get("head_dim", 512)
            d["head_dim"] = d.get("qk_rope_head_dim", 64)
            d.setdefault("scoring_func", "sqrtsoftplus")
            d.setdefault("use_correction_bias", True)
            d.setdefault("sliding_window", 128)
            d.setdefault("routed_scaling_factor", 1.5)
            d.setdefault("router_aux_loss_coef", 0.0)
            d.setdefault("swiglu_limit", 10.0)
            d.setdefault("dense_swiglu_limit", d["swiglu_limit"])
            d.setdefault("intermediate_size", d.get("moe_intermediate_size", 2048))
            if d.get("n_shared_experts") and not d.get("shared_expert_intermediate_size"):
                d["shared_expert_intermediate_size"] = d["n_shared_experts"] * d.get("moe_intermediate_size", 0)
            n = d.get("num_hidden_layers", 43)
            if d.get("compress_ratios") is None:
                # sliding-window-only first layer, then compressed layers alternating 4 and 128
                d["compress_ratios"] = [0] + [4 if i % 2 else 128 for i in range(1, n)]
        if mt == "nemotron_h":
            # one mixer per layer: Mamba2 / attention without rotary embedding / latent MoE / MLP
            lbt = d.get("layers_block_type")
            if lbt is None and d.get("hybrid_override_pattern"):
                lbt = [{"M": "mamba", "*": "attention", "E": "moe", "-": "mlp"}[ch] for ch in d["hybrid_override_pattern"]]
            lbt = list(lbt or ["mamba", "moe", "attention", "moe"])
            d["layers_block_type"] = lbt
            d["num_hidden_layers"] = len(lbt)
            d["use_qk_norm"] = False
            d["no_rope"] = True
            d.setdefault("rms_norm_eps", d.get("layer_norm_epsilon", 1e-5))
            d.setdefault("scoring_func", "sigmoid")
            d.setdefault("use_correction_bias", True)
            d.setdefault("router_aux_loss_coef", 0.0)
            d.setdefault("initializer_range", 0.02)
        extra = {k: d.pop(k) for k in list(d) if k not in known}
        cfg = cls(**d)
        cfg.extra = extra
        return cfg

    @classmethod
    def from_pretrained(cls, path: str) -> "ModelConfig":
        p = path if path.endswith(".json") else os.path.join(path, "config.json")
        with open(p) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self) -> Dict[str, Any]:
        d = asdict(self)
        extra = d.pop("extra", {})
        d.update(extra)
        return d

    def save_pretrained(self, path: str) -> None:
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.to_dict(), f, indent=2)


# Named presets for the benchmark configurations (architecture only; weights are random-init).
PRESETS: Dict[str, Dict[str, Any]] = {
    "tiny-qwen3": dict(model_type="qwen3", vocab_size=1024, hidden_size=256, intermediate_size=768,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=64,
                       rope_theta=1e6, tie_word_embeddings=True, max_position_embeddings=4096),
    "tiny-qwen3-moe": dict(model_type="qwen3_moe", vocab_size=1024, hidden_size=128, intermediate_size=256,
                           num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                           rope_theta=1e6, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=64,
                           norm_topk_prob=True, router_aux_loss_coef=1e-3, tie_word_embeddings=False,
                           max_position_embeddings=4096),
    "small-qwen3": dict(model_type="qwen3", vocab_size=4096, hidden_size=512, intermediate_size=1024,
                        num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                        rope_theta=1e6, tie_word_embeddings=False, max_position_embeddings=8192),
    "small-qwen3-moe": dict(model_type="qwen3_moe", vocab_size=4096, hidden_size=512, intermediate_size=1024,
                            num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=128,
                            rope_theta=1e6, num_experts=8, num_experts_per_tok=2, moe_intermediate_size=256,
                            norm_topk_prob=True, router_aux_loss_coef=1e-3, tie_word_embeddings=False,
                            max_position_embeddings=8192),
    "qwen3-8b": dict(model_type="qwen3", vocab_size=151936, hidden_size=4096, intermediate_size=12288,
                     num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
                     rope_theta=1e6, tie_word_embeddings=False),
    "qwen3-32b": dict(model_type="qwen3", vocab_size=151936, hidden_size=5120, intermediate_size=25600,
                      num_hidden_layers=64, num_attention_heads=64, num_key_value_heads=8, head_dim=128,
                      rope_theta=1e6, tie_word_embeddings=False),
    "qwen3-30b-a3b": dict(model_type="qwen3_moe", vocab_size=151936, hidden_size=2048,
                          intermediate_size=6144, num_hidden_layers=48, num_attention_heads=32,
                          num_key_value_heads=4, head_dim=128, rope_theta=1e6, num_experts=128,
                          num_experts_per_tok=8, moe_intermediate_size=768, norm_topk_prob=True,
                          router_aux_loss_coef=1e-3, tie_word_embeddings=False),
    "tiny-gpt-oss": dict(model_type="gpt_oss", vocab_size=512, hidden_size=64, intermediate_size=64,
                         num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                         num_local_experts=4, num_experts_per_tok=2, sliding_window=8, rope_theta=1e4,
                         max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-deepseek-v3": dict(model_type="deepseek_v3", vocab_size=512, hidden_size=64, intermediate_size=128,
                             num_hidden_layers=3, num_attention_heads=4, num_key_value_heads=4,
                             q_lora_rank=32, kv_lora_rank=24, qk_nope_head_dim=16, qk_rope_head_dim=8,
                             v_head_dim=16, n_routed_experts=8, num_experts_per_tok=2, n_group=4, topk_group=2,
                             n_shared_experts=1, moe_intermediate_size=32, first_k_dense_replace=1,
                             topk_method="noaux_tc", routed_scaling_factor=2.5, norm_topk_prob=True,
                             rope_theta=1e4, max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-glm4-moe": dict(model_type="glm4_moe", vocab_size=512, hidden_size=64, intermediate_size=128,
                          num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                          partial_rotary_factor=0.5, use_qk_norm=True, n_routed_experts=8, num_experts_per_tok=2,
                          n_group=1, topk_group=1, n_shared_experts=1, moe_intermediate_size=32,
                          first_k_dense_replace=1, routed_scaling_factor=1.0, norm_topk_prob=True,
                          rope_theta=1e4, max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-qwen3-5": dict(model_type="qwen3_5", vocab_size=512, hidden_size=64, intermediate_size=128,
                         num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                         linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8,
                         linear_value_head_dim=8, linear_conv_kernel_dim=4, rope_theta=1e4,
                         max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-qwen3-5-moe": dict(model_type="qwen3_5_moe", vocab_size=512, hidden_size=64, intermediate_size=128,
                             num_hidden_layers=4, num_attention_heads=4, num_key_value_heads=2, head_dim=16,
                             linear_num_key_heads=2, linear_num_value_heads=4, linear_key_head_dim=8,
                             linear_value_head_dim=8, linear_conv_kernel_dim=4, num_experts=8,
                             num_experts_per_tok=2, moe_intermediate_size=32, shared_expert_intermediate_size=32,
                             norm_topk_prob=True, rope_theta=1e4, max_position_embeddings=512,
                             tie_word_embeddings=False),
    "tiny-deepseek-v4": dict(model_type="deepseek_v4", vocab_size=512, hidden_size=64, num_hidden_layers=4,
                             num_attention_heads=4, num_key_value_heads=1, head_dim=32, qk_rope_head_dim=8,
                             q_lora_rank=32, o_groups=2, o_lora_rank=16, sliding_window=8, index_n_heads=2,
                             index_head_dim=16, index_topk=3, moe_intermediate_size=32, n_routed_experts=8,
                             n_shared_experts=1, num_experts_per_tok=2, num_hash_layers=1, hc_mult=2,
                             hc_sinkhorn_iters=4, compress_ratios=[0, 4, 128, 4], compress_rope_theta=4e4,
                             rope_theta=1e4, max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-glm5": dict(model_type="glm5", vocab_size=512, hidden_size=64, intermediate_size=128, num_hidden_layers=4,
                      num_attention_heads=4, num_key_value_heads=4, q_lora_rank=32, kv_lora_rank=16,
                      qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, n_routed_experts=8,
                      num_experts_per_tok=2, moe_intermediate_size=32, n_shared_experts=1, first_k_dense_replace=1,
                      n_group=2, topk_group=1, routed_scaling_factor=2.0, norm_topk_prob=True,
                      index_n_heads=2, index_head_dim=16, index_topk=8, index_topk_freq=2,
                      rope_theta=1e4, max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-minimax-m3": dict(model_type="minimax_m3", vocab_size=512, hidden_size=64, num_hidden_layers=4,
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16, rotary_dim=8,
                            dense_intermediate_size=128, intermediate_size=32, shared_intermediate_size=32,
                            num_local_experts=8, num_experts_per_tok=2, n_shared_experts=1, moe_layer_freq=[0, 1, 1, 1],
                            sparse_attention_config=dict(sparse_attention_freq=[0, 1, 0, 1], sparse_block_size=8,
                                                         sparse_topk_blocks=2, sparse_num_index_heads=2,
                                                         sparse_index_dim=16, sparse_init_block=1, sparse_local_block=1),
                            rope_theta=1e4, max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-nemotron-h": dict(model_type="nemotron_h", vocab_size=512, hidden_size=64, intermediate_size=128,
                            layers_block_type=["mamba", "moe", "attention", "mlp", "mamba", "moe"],
                            num_attention_heads=4, num_key_value_heads=2, head_dim=16, mamba_num_heads=8,
                            mamba_head_dim=16, n_groups=2, ssm_state_size=16, conv_kernel=4, chunk_size=32,
                            n_routed_experts=8, num_experts_per_tok=2, moe_intermediate_size=32,
                            moe_shared_expert_intermediate_size=48, moe_latent_size=32, n_group=2, topk_group=1,
                            norm_topk_prob=True, routed_scaling_factor=2.0, layer_norm_epsilon=1e-5,
                            max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-olmo2": dict(model_type="olmo2", vocab_size=512, hidden_size=64, intermediate_size=128,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, rope_theta=1e4,
                       max_position_embeddings=512, tie_word_embeddings=False),
    "tiny-qwen2": dict(model_type="qwen2", vocab_size=512, hidden_size=64, intermediate_size=128,
                       num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2, rope_theta=1e4,
                       max_position_embeddings=512, tie_word_embeddings=True),
    "llama3-8b": dict(model_type="llama", vocab_size=128256, hidden_size=4096, intermediate_size=14336,
                      num_hidden_layers=32, num_attention_heads=32, num_key_value_heads=8,
                      rope_theta=5e5, rms_norm_eps=1e-5, tie_word_embeddings=False, use_qk_norm=False),
}


def preset(name: str, **overrides) -> ModelConfig:
    d = dict(PRESETS[name])
    d.update(overrides)
    return ModelConfig.from_dict(d)
