"""Name / shape transforms between the fused in-memory layout and Hugging Face checkpoints.

In memory: ``self_attn.qkv_proj`` (rows q|k|v), ``mlp.gate_up_proj`` (rows gate|up), MoE experts
stacked as ``mlp.experts.gate_up_proj [E, H, 2I]`` and ``mlp.experts.down_proj [E, I, H]``.
On disk (HF): ``q_proj/k_proj/v_proj``, ``gate_proj/up_proj`` and one tensor per expert.
Counterparts: src/xorl/models/transformers/qwen3/checkpoint_handler.py:23-205 and
qwen3_moe/checkpoint_handler.py.  All FQNs use the ``model.`` prefix of HF causal-LM classes.
"""
from __future__ import annotations

import re
from typing import Dict, Iterator, List, Tuple

import torch


def to_checkpoint_fqn(name: str) -> str:
    """In-memory parameter name -> checkpoint FQN (``model.`` prefix except for ``lm_head``)."""
    return name if name.startswith("lm_head") else "model." + name


def from_checkpoint_fqn(name: str) -> str:
    return name[len("model."):] if name.startswith("model.") else name


class CheckpointHandler:
    def __init__(self, cfg):
        self.cfg = cfg
        self.q, self.kv = cfg.q_size, cfg.kv_size
        self.I = cfg.intermediate_size
        self.moe_I = cfg.moe_intermediate_size

    # ---- export: fused -> HF ------------------------------------------------------------------
    def to_hf(self, name: str, t: torch.Tensor) -> Iterator[Tuple[str, torch.Tensor]]:
        fq = to_checkpoint_fqn(name)
        if ".self_attn.qkv_proj." in fq:
            q, k, v = t.split([self.q, self.kv, self.kv], dim=0)
            for n, part in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                yield fq.replace("qkv_proj", n), part.contiguous()
        elif ".mlp.experts.gate_up_proj" in fq:
            E = t.shape[0]
            base = fq[: fq.index(".experts.")]
            for e in range(E):
                g, u = t[e].split(t.shape[-1] // 2, dim=-1)          # [H, I] each
                yield f"{base}.experts.{e}.gate_proj.weight", g.t().contiguous()
                yield f"{base}.experts.{e}.up_proj.weight", u.t().contiguous()
        elif ".mlp.experts.down_proj" in fq:
            base = fq[: fq.index(".experts.")]
            for e in range(t.shape[0]):
                yield f"{base}.experts.{e}.down_proj.weight", t[e].t().contiguous()   # [H, I]
        elif ".gate_up_proj." in fq:
            g, u = t.split(t.shape[0] // 2, dim=0)
            yield fq.replace("gate_up_proj", "gate_proj"), g.contiguous()
            yield fq.replace("gate_up_proj", "up_proj"), u.contiguous()
        else:
            yield fq, t

    # ---- import: HF -> fused ------------------------------------------------------------------
    def hf_sources(self, name: str) -> List[str]:
        """HF tensor names needed to build in-memory parameter ``name``."""
        fq = to_checkpoint_fqn(name)
        if ".self_attn.qkv_proj." in fq:
            return [fq.replace("qkv_proj", n) for n in ("q_proj", "k_proj", "v_proj")]
        if ".mlp.experts.gate_up_proj" in fq:
            base = fq[: fq.index(".experts.")]
            out = []
            for e in range(self.cfg.num_experts):
                out += [f"{base}.experts.{e}.gate_proj.weight", f"{base}.experts.{e}.up_proj.weight"]
            return out
        if ".mlp.experts.down_proj" in fq:
            base = fq[: fq.index(".experts.")]
            return [f"{base}.experts.{e}.down_proj.weight" for e in range(self.cfg.num_experts)]
        if ".gate_up_proj." in fq:
            return [fq.replace("gate_up_proj", "gate_proj"), fq.replace("gate_up_proj", "up_proj")]
        return [fq]

    def from_hf(self, name: str, parts: List[torch.Tensor]) -> torch.Tensor:
        fq = to_checkpoint_fqn(name)
        if ".mlp.experts.gate_up_proj" in fq:
            E = len(parts) // 2
            return torch.stack([torch.cat([parts[2 * e].t(), parts[2 * e + 1].t()], dim=-1)
                                for e in range(E)])
        if ".mlp.experts.down_proj" in fq:
            return torch.stack([p.t() for p in parts])
        if len(parts) == 1:
            return parts[0]
        return torch.cat(parts, dim=0)


class _RenamingHandler(CheckpointHandler):
    """Base handler plus a table of (in-memory substring, on-disk substring) renames applied after
    the fused-layout transforms."""
    RENAMES: Tuple[Tuple[str, str], ...] = ()

    def _out(self, name: str) -> str:
        for a, b in self.RENAMES:
            name = name.replace(a, b)
        return name

    def _in(self, name: str) -> str:
        for a, b in self.RENAMES:
            name = name.replace(b, a)
        return name

    def to_hf(self, name, t):
        for n, part in super().to_hf(name, t):
            yield self._out(n), part

    def hf_sources(self, name):
        return [self._out(n) for n in super().hf_sources(name)]


class DeepseekV3Handler(_RenamingHandler):
    """DeepSeek-V3 / GLM-4.5 MoE: ``shared_experts`` (plural) on disk, the selection bias stored
    under the router (src/xorl/models/transformers/deepseek_v3/checkpoint_handler.py)."""
    RENAMES = ((".mlp.shared_expert.", ".mlp.shared_experts."),)


class Glm5Handler(DeepseekV3Handler):
    """GLM-5: DeepSeek-style names plus the sparse indexer, whose key LayerNorm is a module on disk
    (``self_attn.indexer.k_norm.weight / .bias``; src/xorl/models/transformers/glm5/indexer.py)."""
    RENAMES = DeepseekV3Handler.RENAMES + ((".indexer.k_norm_weight", ".indexer.k_norm.weight"),
                                           (".indexer.k_norm_bias", ".indexer.k_norm.bias"))


class DeepseekV4Handler(_RenamingHandler):
    """DeepSeek-V4 in the reference's own tensor names: the hyper-connection mixers are flat per-layer
    tensors ``hc_attn_fn / hc_attn_base / hc_attn_scale`` (and ``hc_ffn_*``, ``hc_head_*``), the shared
    expert is ``shared_experts`` (src/xorl/models/transformers/deepseek_v4/modeling_deepseek_v4.py).
    The published checkpoint's packed low-precision expert layout is not parsed here."""
    RENAMES = ((".mlp.shared_expert.", ".mlp.shared_experts."),) + tuple(
        (f"{pre}.{leaf}", f"{pre}_{leaf}") for pre in ("hc_attn", "hc_ffn", "hc_head") for leaf in ("fn", "base", "scale"))


class GptOssHandler(CheckpointHandler):
    """gpt-oss keeps experts stacked on disk, with gate and up columns interleaved, per-expert
    biases, the router under ``mlp.router`` and one sink logit per head
    (src/xorl/models/transformers/gpt_oss/checkpoint_handler.py)."""

    def _disk(self, fq: str) -> str:
        return (fq.replace(".mlp.gate.", ".mlp.router.")
                  .replace(".experts.gate_up_bias", ".experts.gate_up_proj_bias")
                  .replace(".experts.down_bias", ".experts.down_proj_bias"))

    def to_hf(self, name, t):
        fq = to_checkpoint_fqn(name)
        if ".mlp.experts.gate_up_proj" in fq or ".mlp.experts.gate_up_bias" in fq:
            g, u = t.chunk(2, dim=-1)
            yield self._disk(fq), torch.stack([g, u], dim=-1).flatten(-2).contiguous()   # g0 u0 g1 u1 ...
        elif ".mlp.experts." in fq or ".mlp.gate." in fq:
            yield self._disk(fq), t
        else:
            yield from super().to_hf(name, t)

    def hf_sources(self, name):
        fq = to_checkpoint_fqn(name)
        if ".mlp.experts." in fq or ".mlp.gate." in fq:
            return [self._disk(fq)]
        return super().hf_sources(name)

    def from_hf(self, name, parts):
        fq = to_checkpoint_fqn(name)
        if ".mlp.experts.gate_up_proj" in fq or ".mlp.experts.gate_up_bias" in fq:
            t = parts[0]
            return torch.cat([t[..., 0::2], t[..., 1::2]], dim=-1).contiguous()
        if ".mlp.experts." in fq or ".mlp.gate." in fq:
            return parts[0]
        return super().from_hf(name, parts)


class Qwen35Handler(CheckpointHandler):
    """Qwen3.5 / Qwen3.5-MoE.  On disk the linear-attention mixer is ``linear_attn`` with
    ``in_proj_qkv`` (= rows of q, k, v), ``in_proj_z / in_proj_a / in_proj_b``, one ``conv1d.weight``
    [C, 1, K] (= q, k, v taps), ``norm``, ``out_proj``, ``dt_bias``, ``A_log``; gated attention stores
    query and output gate in one ``q_proj`` whose rows alternate per head [query D | gate D]
    (src/xorl/models/transformers/qwen3_5_shared.py:185-300, qwen3_5/modeling_qwen3_5.py).  Export
    buffers the pieces of a fused tensor until the last one has been seen."""
    _SINGLE = {"g_proj": "in_proj_z", "a_proj": "in_proj_a", "b_proj": "in_proj_b", "o_proj": "out_proj"}

    def __init__(self, cfg):
        super().__init__(cfg)
        x = cfg.extra
        self.lk = x["linear_num_key_heads"] * x["linear_key_head_dim"]
        self.lv = x["linear_num_value_heads"] * x["linear_value_head_dim"]
        self.Hq, self.D = cfg.num_attention_heads, cfg.head_dim
        self._pending: Dict[str, Dict[str, torch.Tensor]] = {}

    def _is_linear(self, fq: str) -> bool:
        m = re.search(r"layers\.(\d+)\.", fq)
        return bool(m) and self.cfg.layer_types[int(m.group(1))] == "linear_attention"

    # ---- export ---------------------------------------------------------------------------------
    def to_hf(self, name, t):
        fq = to_checkpoint_fqn(name)
        if ".self_attn." in fq and self._is_linear(fq):
            base, leaf = fq.split(".self_attn.", 1)
            la = base + ".linear_attn."
            part = leaf.split(".")[0]
            if part in ("q_proj", "k_proj", "v_proj") or part in ("q_conv1d", "k_conv1d", "v_conv1d"):
                conv = "conv1d" in part
                key = la + ("conv1d.weight" if conv else "in_proj_qkv.weight")
                buf = self._pending.setdefault(key, {})
                buf[part[0]] = t.unsqueeze(1) if conv else t
                if len(buf) == 3:
                    del self._pending[key]
                    yield key, torch.cat([buf["q"], buf["k"], buf["v"]], dim=0).contiguous()
            elif part in self._SINGLE:
                yield la + leaf.replace(part, self._SINGLE[part], 1), t
            elif part == "o_norm_weight":
                yield la + "norm.weight", t
            else:                                                   # dt_bias, A_log
                yield la + leaf, t
            return
        if ".self_attn.qkv_proj.weight" in fq or ".self_attn.out_gate.weight" in fq:
            base = fq.split(".self_attn.", 1)[0] + ".self_attn."
            buf = self._pending.setdefault(base, {})
            buf["qkv" if "qkv_proj" in fq else "gate"] = t
            if len(buf) == 2:
                del self._pending[base]
                q, k, v = buf["qkv"].split([self.q, self.kv, self.kv], dim=0)
                qg = torch.cat([q.view(self.Hq, self.D, -1), buf["gate"].view(self.Hq, self.D, -1)], dim=1)
                yield base + "q_proj.weight", qg.reshape(2 * self.q, -1).contiguous()
                yield base + "k_proj.weight", k.contiguous()
                yield base + "v_proj.weight", v.contiguous()
            return
        if ".mlp.shared_expert_gate." in fq:
            yield fq, t
            return
        yield from super().to_hf(name, t)

    # ---- import ---------------------------------------------------------------------------------
    def hf_sources(self, name):
        fq = to_checkpoint_fqn(name)
        if ".self_attn." in fq and self._is_linear(fq):
            base, leaf = fq.split(".self_attn.", 1)
            la = base + ".linear_attn."
            part = leaf.split(".")[0]
            if part in ("q_proj", "k_proj", "v_proj"):
                return [la + "in_proj_qkv.weight"]
            if "conv1d" in part:
                return [la + "conv1d.weight"]
            if part in self._SINGLE:
                return [la + leaf.replace(part, self._SINGLE[part], 1)]
            if part == "o_norm_weight":
                return [la + "norm.weight"]
            return [la + leaf]
        if ".self_attn.out_gate.weight" in fq:
            return [fq.replace("out_gate", "q_proj")]
        return super().hf_sources(name)

    def from_hf(self, name, parts):
        fq = to_checkpoint_fqn(name)
        if ".self_attn." in fq and self._is_linear(fq):
            part = fq.split(".self_attn.", 1)[1].split(".")[0]
            t = parts[0]
            if part in ("q_proj", "k_proj", "v_proj") or "conv1d" in part:
                lo = {"q": 0, "k": self.lk, "v": 2 * self.lk}[part[0]]
                hi = lo + (self.lv if part[0] == "v" else self.lk)
                t = t[lo:hi]
                return (t.squeeze(1) if "conv1d" in part else t).contiguous()
            return t
        if ".self_attn.out_gate.weight" in fq:
            return parts[0].view(self.Hq, 2, self.D, -1)[:, 1].reshape(self.q, -1).contiguous()
        if ".self_attn.qkv_proj.weight" in fq:
            q = parts[0].view(self.Hq, 2, self.D, -1)[:, 0].reshape(self.q, -1)
            return torch.cat([q, parts[1], parts[2]], dim=0).contiguous()
        return super().from_hf(name, parts)


class NemotronHHandler(CheckpointHandler):
    """Nemotron-H: the module tree is ``backbone.*`` on disk (``embeddings``, ``norm_f``, one
    ``mixer`` per layer), attention projections are separate, the depthwise convolution is stored as
    ``conv1d.weight [C, 1, K]`` / ``conv1d.bias``, and the non-gated experts are one
    ``up_proj [I, latent]`` / ``down_proj [latent, I]`` pair per expert
    (src/xorl/models/transformers/nemotron_h/checkpoint_handler.py)."""
    _LEAF = (("mixer.conv1d_weight", "mixer.conv1d.weight"), ("mixer.conv1d_bias", "mixer.conv1d.bias"),
             ("mixer.norm_weight", "mixer.norm.weight"), ("mixer.shared_expert.", "mixer.shared_experts."))

    def _disk(self, name: str) -> str:
        fq = to_checkpoint_fqn(name)
        if fq.startswith("model."):
            fq = "backbone." + fq[len("model."):]
        fq = fq.replace("backbone.embed_tokens.", "backbone.embeddings.")
        if fq.startswith("backbone.norm."):
            fq = fq.replace("backbone.norm.", "backbone.norm_f.")
        for a, b in self._LEAF:
            fq = fq.replace(a, b)
        return fq

    def to_hf(self, name, t):
        fq = self._disk(name)
        if ".mixer.qkv_proj." in fq:
            q, k, v = t.split([self.q, self.kv, self.kv], dim=0)
            for n, part in (("q_proj", q), ("k_proj", k), ("v_proj", v)):
                yield fq.replace("qkv_proj", n), part.contiguous()
        elif fq.endswith(".mixer.experts.gate_up_proj"):
            base = fq[: fq.index(".experts.")]
            for e in range(t.shape[0]):
                yield f"{base}.experts.{e}.up_proj.weight", t[e].t().contiguous()
        elif fq.endswith(".mixer.experts.down_proj"):
            base = fq[: fq.index(".experts.")]
            for e in range(t.shape[0]):
                yield f"{base}.experts.{e}.down_proj.weight", t[e].t().contiguous()
        elif fq.endswith(".mixer.conv1d.weight"):
            yield fq, t.unsqueeze(1).contiguous()
        else:
            yield fq, t

    def hf_sources(self, name):
        fq = self._disk(name)
        if ".mixer.qkv_proj." in fq:
            return [fq.replace("qkv_proj", n) for n in ("q_proj", "k_proj", "v_proj")]
        if fq.endswith(".mixer.experts.gate_up_proj") or fq.endswith(".mixer.experts.down_proj"):
            base = fq[: fq.index(".experts.")]
            leaf = "up_proj" if fq.endswith("gate_up_proj") else "down_proj"
            return [f"{base}.experts.{e}.{leaf}.weight" for e in range(self.cfg.num_experts)]
        return [fq]

    def from_hf(self, name, parts):
        fq = self._disk(name)
        if fq.endswith(".mixer.experts.gate_up_proj") or fq.endswith(".mixer.experts.down_proj"):
            return torch.stack([p.t() for p in parts])
        if fq.endswith(".mixer.conv1d.weight"):
            return parts[0].squeeze(1).contiguous()
        return parts[0] if len(parts) == 1 else torch.cat(parts, dim=0)


class MiniMaxM3Handler(CheckpointHandler):
    """MiniMax-M3 text weights: on disk the MoE block is ``block_sparse_moe`` with per-expert
    ``w1`` (gate), ``w3`` (up), ``w2`` (down), the selection bias directly under the block, and
    ``shared_experts`` (plural); dense layers keep ``mlp.gate_proj / up_proj / down_proj``
    (src/xorl/models/transformers/minimax_m3/checkpoint_handler.py).  Keys of a multimodal checkpoint
    carry a ``language_model.`` prefix, which ``normalize_key`` strips before lookup."""

    @staticmethod
    def normalize_key(key: str) -> str:
        for pre, new in (("model.language_model.model.", "model."), ("language_model.model.", "model."),
                         ("model.language_model.lm_head.", "lm_head."), ("language_model.lm_head.", "lm_head."),
                         ("model.language_model.", ""), ("language_model.", "")):
            if key.startswith(pre):
                return new + key[len(pre):]
        return key

    def _is_moe(self, fq: str) -> bool:
        m = re.search(r"layers\.(\d+)\.", fq)
        return bool(m) and self.cfg.layer_is_moe(int(m.group(1)))

    def _disk(self, fq: str) -> str:
        if ".mlp." in fq and self._is_moe(fq):
            fq = fq.replace(".mlp.", ".block_sparse_moe.")
            fq = fq.replace(".block_sparse_moe.gate.e_score_correction_bias", ".block_sparse_moe.e_score_correction_bias")
            fq = fq.replace(".block_sparse_moe.shared_expert.", ".block_sparse_moe.shared_experts.")
        return fq

    def to_hf(self, name, t):
        fq = to_checkpoint_fqn(name)
        if ".mlp.experts.gate_up_proj" in fq:
            base = self._disk(fq[: fq.index(".experts.")] + ".")[:-1]
            for e in range(t.shape[0]):
                g, u = t[e].split(t.shape[-1] // 2, dim=-1)
                yield f"{base}.experts.{e}.w1.weight", g.t().contiguous()
                yield f"{base}.experts.{e}.w3.weight", u.t().contiguous()
        elif ".mlp.experts.down_proj" in fq:
            base = self._disk(fq[: fq.index(".experts.")] + ".")[:-1]
            for e in range(t.shape[0]):
                yield f"{base}.experts.{e}.w2.weight", t[e].t().contiguous()
        else:
            for n, part in super().to_hf(name, t):
                yield self._disk(n), part

    def hf_sources(self, name):
        fq = to_checkpoint_fqn(name)
        if ".mlp.experts.gate_up_proj" in fq or ".mlp.experts.down_proj" in fq:
            base = self._disk(fq[: fq.index(".experts.")] + ".")[:-1]
            ws = ("w1", "w3") if "gate_up_proj" in fq else ("w2",)
            return [f"{base}.experts.{e}.{w}.weight" for e in range(self.cfg.num_experts) for w in ws]
        return [self._disk(n) for n in super().hf_sources(name)]


def get_checkpoint_handler(cfg) -> CheckpointHandler:
    mt = getattr(cfg, "model_type", "")
    if mt == "minimax_m3":
        return MiniMaxM3Handler(cfg)
    if mt == "nemotron_h":
        return NemotronHHandler(cfg)
    if mt in ("qwen3_5", "qwen3_5_moe", "qwen3_next"):
        return Qwen35Handler(cfg)
    if mt == "gpt_oss":
        return GptOssHandler(cfg)
    if mt == "glm5":
        return Glm5Handler(cfg)
    if mt == "deepseek_v4":
        return DeepseekV4Handler(cfg)
    if mt in ("deepseek_v3", "glm4_moe"):
        return DeepseekV3Handler(cfg)
    return CheckpointHandler(cfg)
