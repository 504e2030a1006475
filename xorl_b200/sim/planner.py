"""Step-time and memory model of one training step under a parallel layout.

The model is a roofline with calibrated efficiencies: GEMM and attention FLOPs over a measured
tensor throughput, optimizer and elementwise bytes over measured HBM bandwidth, collective bytes
over measured NVLink bandwidth with a configurable overlap factor, and the pipeline bubble from
the schedule's analytic formula.  A *calibration pack* (a JSON file or dict) overrides the default
efficiencies with ratios measured on the target machine; ``default_b200_pack`` carries the ratios
measured for this framework's kernels on one B200 (src/xorl/sim/scenario_planner.py, calibration/).
"""
from __future__ import annotations

import itertools
import json
import math
from dataclasses import asdict, dataclass, field
from typing import Dict, Iterable, List, Optional

from ..models.config import ModelConfig
from ..parallel.pp_schedules import analytic_bubble_fraction
from ..utils.count_flops import model_flops_per_token


@dataclass
class HardwareSpec:
    name: str = "B200"
    hbm_gb: float = 192.0                   # 183,359 MiB reported by the driver, in decimal GB
    hbm_gbs: float = 6538.0                 # measured copy bandwidth
    bf16_tflops: float = 1360.0             # measured sustained cuBLAS bf16
    nvlink_gbs: float = 770.0               # per direction per GPU (measured peer copy)
    allreduce_busbw_gbs: float = 725.0      # 8-rank bus bandwidth at 1 GiB
    internode_gbs: float = 50.0             # per GPU, for layouts that leave the box
    gpus_per_node: int = 8

    @classmethod
    def from_measured(cls, path: str) -> "HardwareSpec":
        with open(path) as f:
            m = json.load(f)
        return cls(name=m.get("chip", "B200"), hbm_gbs=m.get("hbm_gbs", cls.hbm_gbs),
                   bf16_tflops=m.get("bf16_tflops_sustained", m.get("bf16_tflops", cls.bf16_tflops)))


def default_b200_pack() -> Dict[str, float]:
    return {
        "gemm_eff": 0.90,            # tcgen05 pair GEMM relative to cuBLAS sustained
        "attn_fwd_tflops": 400.0,    # tcgen05 flash attention forward, causal, D=128
        "attn_bwd_tflops": 200.0,
        "optimizer_eff": 0.93,       # AdamW kernel relative to copy bandwidth
        "elementwise_bytes_per_token_per_layer_per_hidden": 44.0,   # norms, rope, swiglu, residuals (bf16)
        "comm_overlap": 0.85,        # fraction of ZeRO gather / reduce-scatter hidden behind compute
        "tp_overlap": 0.0,
        "ep_overlap": 0.3,
        "launch_overhead_ms_per_layer": 0.05,
        "moe_gemm_eff": 0.6,
    }


@dataclass
class ParallelLayout:
    dp_shard: int = 1
    dp_replicate: int = 1
    tp: int = 1
    pp: int = 1
    cp: int = 1
    ep: int = 1
    pp_schedule: str = "1f1b"
    virtual_stages: int = 1
    micro_batches: int = 1
    recompute: bool = True

    @property
    def world(self) -> int:
        return self.dp_shard * self.dp_replicate * self.tp * self.pp * self.cp

    def tag(self) -> str:
        parts = [f"fsdp{self.dp_shard}"]
        for n, v in (("hsdp", self.dp_replicate), ("tp", self.tp), ("pp", self.pp), ("cp", self.cp), ("ep", self.ep)):
            if v > 1:
                parts.append(f"{n}{v}")
        return "-".join(parts)


@dataclass
class Estimate:
    layout: ParallelLayout
    step_ms: float
    tokens_per_s: float
    mfu: float
    memory_gb: float
    fits: bool
    breakdown_ms: Dict[str, float] = field(default_factory=dict)
    memory_breakdown_gb: Dict[str, float] = field(default_factory=dict)

    def to_dict(self):
        d = asdict(self)
        d["layout"] = self.layout.tag()
        return d


def _params(cfg: ModelConfig):
    total = cfg.num_parameters(include_embeddings=True)
    expert = 0
    for i in range(cfg.num_hidden_layers):
        if cfg.layer_is_moe(i):
            expert += cfg.num_experts * 3 * cfg.hidden_size * cfg.moe_intermediate_size
    return total, expert


def estimate(cfg: ModelConfig, layout: ParallelLayout, seq_len: int, micro_batch_tokens: Optional[int] = None,
             hw: Optional[HardwareSpec] = None, pack: Optional[Dict[str, float]] = None,
             doc_lens: Optional[List[int]] = None, optimizer_bytes_per_param: float = 30.0) -> Estimate:
    """One optimizer step; every data-parallel rank processes ``micro_batches`` micro-batches of
    ``micro_batch_tokens`` tokens (default ``seq_len``), sequences split ``cp`` ways."""
    hw = hw or HardwareSpec()
    p = dict(default_b200_pack())
    p.update(pack or {})
    L, H = cfg.num_hidden_layers, cfg.hidden_size
    tok_mb = micro_batch_tokens or seq_len
    n_mb = layout.micro_batches
    tokens_rank = tok_mb * n_mb / layout.cp               # tokens whose activations live on a rank
    doc_lens = doc_lens or [seq_len]
    total_p, expert_p = _params(cfg)
    dense_p = total_p - expert_p

    # ---- compute ------------------------------------------------------------------------------
    fl_tok = model_flops_per_token(cfg, None, True, layout.recompute)
    attn_per_tok = model_flops_per_token(cfg, doc_lens, False, False) - model_flops_per_token(cfg, None, False, False)
    shard = layout.tp * layout.pp
    gemm_ms = fl_tok * tokens_rank / shard / (hw.bf16_tflops * 1e12 * p["gemm_eff"]) * 1e3
    if cfg.is_moe:
        gemm_ms /= max(p["moe_gemm_eff"] / p["gemm_eff"], 1e-3) ** (expert_p / max(total_p, 1))
    fwd_passes = 2.0 if layout.recompute else 1.0
    attn_ms = attn_per_tok * tokens_rank / shard * (fwd_passes / (p["attn_fwd_tflops"] * 1e12)
                                                    + 2.5 / (p["attn_bwd_tflops"] * 1e12)) * 1e3
    elem_bytes = p["elementwise_bytes_per_token_per_layer_per_hidden"] * tokens_rank * (L / layout.pp) * H \
        * (3.0 if layout.recompute else 2.0) / layout.tp
    elem_ms = elem_bytes / (hw.hbm_gbs * 1e9) * 1e3
    launch_ms = p["launch_overhead_ms_per_layer"] * (L / layout.pp) * n_mb

    # ---- optimizer ------------------------------------------------------------------------------
    shard_ways_dense = layout.dp_shard * layout.cp * layout.tp * layout.pp
    shard_ways_exp = max(1, shard_ways_dense)             # experts: ep x (dp_shard*cp/ep) ways in total
    local_params = dense_p / shard_ways_dense + expert_p / shard_ways_exp
    opt_ms = local_params * optimizer_bytes_per_param / (hw.hbm_gbs * 1e9 * p["optimizer_eff"]) * 1e3

    # ---- communication ------------------------------------------------------------------------
    zero_group = layout.dp_shard * layout.cp
    stage_params = (dense_p + expert_p / max(1, layout.ep)) / (layout.tp * layout.pp)
    ag_passes = (2.0 if layout.recompute else 1.0) + 1.0   # forward (+ recompute) and backward gathers
    zero_bytes = stage_params * 2 * (zero_group - 1) / zero_group * (ag_passes + 1.0) * n_mb
    bw = hw.nvlink_gbs if layout.world <= hw.gpus_per_node else hw.internode_gbs
    zero_ms = zero_bytes / (bw * 1e9) * 1e3 * (1.0 - p["comm_overlap"]) if zero_group > 1 else 0.0
    tp_ms = 0.0
    if layout.tp > 1:
        per_layer = 4 * tokens_rank * H * 2 * 2 * (layout.tp - 1) / layout.tp      # 2 fwd + 2 bwd all-reduces
        tp_ms = per_layer * (L / layout.pp) * (1.5 if layout.recompute else 1.0) / (hw.allreduce_busbw_gbs * 1e9) \
            * 1e3 * (1.0 - p["tp_overlap"])
    cp_ms = 0.0
    if layout.cp > 1:
        kv = 2 * tokens_rank * cfg.kv_size * 2 * (layout.cp - 1)
        cp_ms = kv * (L / layout.pp) * 3 / (bw * 1e9) * 1e3 * 0.5
    ep_ms = 0.0
    if cfg.is_moe and layout.ep > 1:
        moe_layers = sum(cfg.layer_is_moe(i) for i in range(L)) / layout.pp
        a2a = tokens_rank * cfg.num_experts_per_tok * H * 2 * (layout.ep - 1) / layout.ep
        ep_ms = a2a * 4 * moe_layers * (1.5 if layout.recompute else 1.0) / (bw * 1e9) * 1e3 * (1.0 - p["ep_overlap"])
    hsdp_ms = 0.0
    if layout.dp_replicate > 1:
        hsdp_ms = local_params * 4 * 2 / (hw.allreduce_busbw_gbs * 1e9) * 1e3
    compute_ms = gemm_ms + attn_ms + elem_ms + launch_ms
    bubble = analytic_bubble_fraction(layout.pp_schedule, layout.pp, n_mb, layout.virtual_stages) if layout.pp > 1 else 0.0
    pipe_ms = (compute_ms + tp_ms + cp_ms + ep_ms) / max(1e-6, 1.0 - bubble)
    step_ms = pipe_ms + zero_ms + opt_ms + hsdp_ms

    # ---- memory ---------------------------------------------------------------------------------
    mem = {
        "master_and_states": local_params * 12 / 1e9,
        "compute_shard_and_grads": local_params * (2 + 4) / 1e9,
        # gathered copies exist only when parameters are actually sharded over a group
        "gathered_units": (3 * (stage_params / max(1, L / layout.pp)) * (2 + 4) / 1e9) if zero_group > 1 else
                          (stage_params / max(1, L / layout.pp)) * 4 / 1e9,
        "root_unit": (2 * cfg.vocab_size * H * (2 + 4) / 1e9 / layout.tp / (1 if layout.pp == 1 else 2))
        if zero_group > 1 else 0.0,
    }
    act_per_tok_layer = (2 * H * 2) if layout.recompute else (34 * H * 2 + 2 * cfg.intermediate_size * 2) / layout.tp
    inflight = min(n_mb, layout.pp) if layout.pp > 1 else 1
    mem["activations"] = act_per_tok_layer * (tok_mb / layout.cp) * (L / layout.pp) * inflight / 1e9
    mem["layer_working_set"] = (40 * H + 6 * cfg.intermediate_size) * (tok_mb / layout.cp) * 2 / layout.tp / 1e9
    mem["logits_chunk"] = 1024 * cfg.vocab_size * 2 * 2 / 1e9 / layout.tp
    memory_gb = sum(mem.values()) * 1.03 + 1.5
    tokens_step = tok_mb * n_mb * layout.dp_shard * layout.dp_replicate
    tps = tokens_step / (step_ms / 1e3)
    useful = model_flops_per_token(cfg, doc_lens, True, False) * tokens_step
    mfu = useful / (step_ms / 1e3) / (layout.world * 2250e12)
    return Estimate(layout, step_ms, tps, mfu, memory_gb, memory_gb <= hw.hbm_gb * 0.95,
                    {"gemm": gemm_ms, "attention": attn_ms, "elementwise": elem_ms, "launch": launch_ms,
                     "optimizer": opt_ms, "zero_exposed": zero_ms, "tp": tp_ms, "cp": cp_ms, "ep": ep_ms,
                     "hsdp": hsdp_ms, "pipeline_bubble": pipe_ms - (compute_ms + tp_ms + cp_ms + ep_ms)}, mem)


def enumerate_layouts(cfg: ModelConfig, world: int, seq_len: int, max_tp: int = 8, micro_batches: int = 1,
                      gpus_per_node: int = 8) -> Iterable[ParallelLayout]:
    def divisors(n):
        return [d for d in range(1, n + 1) if n % d == 0]
    for tp, pp, cp in itertools.product(divisors(world), repeat=3):
        if tp * pp * cp > world or world % (tp * pp * cp):
            continue
        if tp > min(max_tp, gpus_per_node) or cfg.num_attention_heads % tp or cfg.num_key_value_heads % tp:
            continue
        if cfg.num_hidden_layers % pp or (cp > 1 and seq_len % (2 * cp)):
            continue
        dp = world // (tp * pp * cp)
        eps = [e for e in divisors(dp * cp) if cfg.is_moe and cfg.num_experts % e == 0] or [1]
        for ep in (eps if cfg.is_moe else [1]):
            n_mb = max(micro_batches, 2 * pp if pp > 1 else micro_batches)
            yield ParallelLayout(dp_shard=dp, tp=tp, pp=pp, cp=cp, ep=ep, micro_batches=n_mb,
                                 pp_schedule="1f1b" if pp > 1 else "1f1b")


def plan(cfg: ModelConfig, world: int, seq_len: int, hw: Optional[HardwareSpec] = None,
         pack: Optional[Dict[str, float]] = None, top: int = 5, **kw) -> List[Estimate]:
    """Feasible layouts for ``world`` GPUs ranked by tokens/s."""
    ests = [estimate(cfg, lay, seq_len, hw=hw, pack=pack) for lay in enumerate_layouts(cfg, world, seq_len, **kw)]
    ests = [e for e in ests if e.fits] or sorted(ests, key=lambda e: e.memory_gb)[:top]
    return sorted(ests, key=lambda e: -e.tokens_per_s)[:top]
