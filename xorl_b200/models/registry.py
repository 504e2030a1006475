"""Architecture name / model_type -> model class (cf. src/xorl/models/registry.py:20-69)."""
from __future__ import annotations

from typing import Callable, Dict

MODEL_REGISTRY: Dict[str, Callable] = {}


def register(*names: str):
    def deco(fn):
        for n in names:
            MODEL_REGISTRY[n] = fn
        return fn
    return deco


def _decoder():
    from .decoder import DecoderLM
    return DecoderLM


for _n in ("qwen3", "Qwen3ForCausalLM", "qwen2", "Qwen2ForCausalLM", "llama", "LlamaForCausalLM",
           "olmo2", "Olmo2ForCausalLM", "qwen3_moe", "Qwen3MoeForCausalLM", "glm4_moe",
           "Glm4MoeForCausalLM", "gpt_oss", "GptOssForCausalLM", "deepseek_v3",
           "DeepseekV3ForCausalLM", "qwen3_5", "qwen3_5_moe", "qwen3_next", "Qwen3NextForCausalLM",
           "Qwen3_5ForCausalLM", "Qwen3_5MoeForCausalLM", "nemotron_h", "NemotronHForCausalLM",
           "glm5", "Glm5ForCausalLM", "GlmMoeDsaForCausalLM", "deepseek_v4", "DeepseekV4ForCausalLM",
           "minimax_m3", "MiniMaxM3SparseForCausalLM", "MiniMaxM3SparseForConditionalGeneration"):
    MODEL_REGISTRY[_n] = _decoder

# model_type -> reason, for architectures that are known but not built (none at present): asking for
# one fails loudly instead of training a different architecture under the same name.
UNSUPPORTED: Dict[str, str] = {}


def get_model_class(cfg):
    for key in [cfg.model_type] + list(cfg.architectures or []):
        if key in MODEL_REGISTRY:
            return MODEL_REGISTRY[key]()
    if cfg.model_type in UNSUPPORTED:
        raise NotImplementedError(f"model_type {cfg.model_type!r} needs {UNSUPPORTED[cfg.model_type]}, "
                                  f"which this framework does not implement")
    raise KeyError(f"no model registered for model_type={cfg.model_type!r} "
                   f"architectures={cfg.architectures}")
