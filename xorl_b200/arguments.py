"""Configuration: nested dataclasses <-> YAML / JSON with ``--section.field value`` overrides.

Same sections (``model: data: train: lora: distill:``), key names and defaults as the reference
(src/xorl/arguments.py:237-2422) so that its example configs load unchanged.  CLI beats YAML,
unknown keys are errors (src/xorl/arguments.py:2284-2302), derived sizes and cross-field validation
live in ``__post_init__`` (src/xorl/arguments.py:1649-1829), the resolved config is written to
``{output_dir}/xorl_cli.yaml`` (src/xorl/arguments.py:2354-2365).
"""
from __future__ import annotations

import json
import os
import sys
import types
from dataclasses import MISSING, asdict, dataclass, field, fields, is_dataclass
from typing import Any, Dict, List, Literal, Optional, Union, get_args, get_origin, get_type_hints

import yaml

PP_SCHEDULES = ("gpipe", "1f1b", "interleaved1f1b", "interleavedzerobubble", "zbvzerobubble",
                "dualpipev")


@dataclass
class ModelArguments:
    config_path: Optional[str] = None
    model_path: Optional[str] = None
    tokenizer_path: Optional[str] = None
    foundation: Dict[str, Any] = field(default_factory=dict)
    encoders: Dict[str, Any] = field(default_factory=dict)
    attn_implementation: Optional[str] = None
    flash_attention_deterministic: bool = False
    moe_implementation: Optional[str] = None
    moe_routing_weights_before_down: Literal["auto", "true", "false"] = "auto"
    ep_dispatch: str = "alltoall"
    train_router: bool = False
    freeze_router: bool = False
    record_routing_weights: bool = True
    deepep_buffer_size_gb: float = 2.0
    deepep_num_sms: int = 20
    deepep_async_combine: bool = False
    alltoall_combine_hidden_chunk_size: int = 0
    basic_modules: Optional[List[str]] = field(default_factory=list)
    merge_qkv: bool = True
    rmsnorm_mode: Optional[str] = None
    qwen35_rmsnorm_family: Optional[str] = None
    router_fp32: Optional[bool] = None
    lm_head_fp32: Optional[bool] = None
    activation_native: bool = False
    rope_native: Optional[bool] = None
    rope_class_b: Optional[bool] = None
    attention_cast_bf16: bool = False
    sparse_mla_enabled: Optional[bool] = None
    sparse_mla_backend: Literal["auto", "tilelang", "flashmla", "native"] = "auto"

    def __post_init__(self):
        if self.config_path is None and self.model_path is None:
            return
        if self.config_path is None:
            self.config_path = self.model_path
        if self.tokenizer_path is None:
            self.tokenizer_path = self.config_path
        if self.ep_dispatch not in ("alltoall", "deepep", "fused"):
            raise ValueError(f"ep_dispatch must be alltoall|deepep|fused, got {self.ep_dispatch!r}")
        if self.train_router and self.freeze_router:
            raise ValueError("train_router and freeze_router are mutually exclusive")


@dataclass
class DataArguments:
    datasets: Optional[List[Dict[str, Any]]] = field(default_factory=list)
    test_datasets: Optional[List[Dict[str, Any]]] = field(default_factory=list)
    dataset_prepared_path: str = "last_prepared_dataset"
    shuffle_merged_datasets: Optional[bool] = True
    shuffle_before_merging_datasets: Optional[bool] = True
    push_dataset_to_hub: Optional[str] = None
    hf_use_auth_token: Optional[bool] = None
    skip_prepare_dataset: Optional[bool] = False
    is_preprocess: Optional[bool] = False
    num_dataset_shards_to_save: Optional[int] = None
    dataset_shard_num: Optional[int] = None
    dataset_shard_idx: Optional[int] = None
    val_set_size: Optional[float] = None
    dataset_num_proc: Optional[int] = None
    sample_packing_method: Optional[str] = "sequential"
    sample_packing_group_size: Optional[int] = 100000
    sample_packing_bin_size: Optional[int] = 100000
    sample_packing_sequentially: Optional[bool] = None
    sample_packing_mp_start_method: Optional[str] = None
    eval_sample_packing: Optional[bool] = None
    sample_packing_sequence_len: Optional[int] = 32000
    select_columns: Optional[List[str]] = None
    dataloader_pin_memory: Optional[bool] = True
    dataloader_num_workers: Optional[int] = 8
    dataloader_prefetch_factor: Optional[int] = 2
    dataloader_drop_last: Optional[bool] = True
    pad_to_multiple_of: Optional[int] = 128
    fa_max_length_bucket: int = 0


@dataclass
class TrainingArguments:
    output_dir: str = "outputs"
    lr: float = 5e-5
    lr_min: float = 1e-7
    lr_start: float = 0.0
    weight_decay: float = 0
    cautious_weight_decay: bool = False
    no_decay_modules: List[str] = field(default_factory=list)
    no_decay_params: List[str] = field(default_factory=list)
    optimizer: Literal["adamw", "anyprecision_adamw", "sgd", "signsgd", "distsignsgd", "muon"] = "adamw"
    optimizer_dtype: Literal["fp32", "bf16"] = "bf16"
    anyprecision_adamw_denominator_chunk_size: int = 0
    anyprecision_adamw_reuse_grad_for_momentum: bool = False
    anyprecision_adamw_state_cpu_offload: bool = False
    muon_lr: float = 0.02
    muon_momentum: float = 0.95
    muon_nesterov: bool = True
    muon_ns_steps: int = 5
    muon_adjust_lr_fn: Optional[str] = None
    muon_ns_algorithm: Literal["gram_newton_schulz", "newton_schulz"] = "gram_newton_schulz"
    muon_ns_use_quack_kernels: bool = True
    muon_gram_ns_num_restarts: int = 1
    muon_gram_ns_restart_iterations: Optional[List[int]] = None
    muon_grouped_gram_ns_fp32_byte_limit: int = 536870912
    muon_fallback_optimizer: Literal["adamw", "anyprecision_adamw"] = "adamw"
    muon_grad_dtype: Optional[str] = None
    muon_update_dtype: Optional[str] = None
    muon_force_momentum_path: bool = False
    muon_distributed_mode: Literal["shard_local", "full_gradient"] = "shard_local"
    max_grad_norm: float = 1.0
    softmax_auxiliary_loss: bool = False
    auxiliary_loss_multiplier: float = 1e-5
    moe_global_load_balancing: bool = False
    ce_mode: Optional[str] = None
    ce_num_chunks: int = 8
    micro_batch_size: int = 1
    gradient_accumulation_steps: int = 1
    defer_grad_sync_in_accumulation: bool = False
    num_train_epochs: int = 1
    lr_warmup_ratio: float = 0
    lr_decay_style: str = "constant"
    lr_decay_ratio: float = 1.0
    enable_mixed_precision: bool = True
    fsdp_reduce_dtype: Literal["fp32", "bf16"] = "fp32"
    skip_param_upcast: bool = False
    fp8_cfg: Optional[Dict[str, Any]] = None
    enable_fp8_training: bool = False
    enable_qarl: bool = False
    qarl_quant_cfg: Optional[Union[str, Dict[str, Any]]] = None
    qarl_calib_data: Optional[str] = None
    qarl_calib_size: int = 0
    qarl_quant_sequence_length: Optional[int] = None
    qarl_sync_format: Literal["fp8", "nvfp4", "bf16"] = "fp8"
    qarl_target_modules: Optional[List[str]] = None
    qarl_exclude_modules: Optional[List[str]] = None
    fp8_training_num_first_layers_bf16: int = 0
    fp8_training_num_last_layers_bf16: int = 0
    fp8_training_allow_blackwell: bool = False
    fp8_training_blackwell_validation_artifact: Optional[str] = None
    fp8_training_block_size: int = 128
    fp8_training_backward: Literal["fp8", "bf16"] = "fp8"
    fp8_training_smoothquant_alpha: Optional[float] = None
    fp8_training_lm_head_smoothquant_alpha: Optional[float] = None
    fp8_training_activation_amax_scale: float = 1.0
    fp8_training_weight_amax_scale: float = 1.0
    fp8_training_correction_mode: Literal["none", "residual"] = "none"
    fp8_training_module_overrides: Optional[Dict[str, Any]] = None
    fp8_training_moe_grouped_backend: Literal["triton_grouped", "deep_gemm", "native"] = "triton_grouped"
    fp8_training_target_modules: Optional[List[str]] = None
    fp8_training_exclude_modules: Optional[List[str]] = None
    fp8_training_allow_bf16_fallback: bool = False
    enable_gradient_checkpointing: bool = True
    enable_reentrant: bool = False
    gradient_checkpointing_method: Optional[str] = None
    moe_checkpoint_method: Optional[str] = None
    enable_full_shard: bool = True
    enable_forward_prefetch: bool = True
    enable_backward_prefetch: Optional[bool] = None
    enable_activation_offload: bool = False
    activation_gpu_limit: float = 0.0
    activation_offload_prefetch_count: int = 2
    init_device: Literal["cpu", "cuda", "meta"] = "cuda"
    load_weights_mode: Literal["grouped", "all_ranks", "broadcast", "skip"] = "grouped"
    enable_full_determinism: bool = False
    high_precision_bf16: bool = False
    allow_cuda_launch_blocking: bool = False
    prewarm_cuda_blas: bool = False
    empty_cache_steps: int = 500
    gc_steps: int = 500
    data_parallel_mode: Literal["none", "ddp", "fsdp2"] = "fsdp2"
    data_parallel_replicate_size: int = -1
    data_parallel_shard_size: int = -1
    expert_parallel_size: int = 1
    ep_intranode: bool = True
    ep_outside: Optional[bool] = None
    ulysses_parallel_size: int = 1
    tensor_parallel_size: int = 1
    # sequence-parallel activations between the tensor-parallel regions: all-gather -> GEMM and
    # GEMM -> reduce-scatter run as single kernels over NVLink peer memory
    tensor_parallel_sequence_parallel: bool = False
    lm_head_tensor_parallel_size: int = 1
    ringattn_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    pipeline_parallel_schedule: str = "1F1B"
    pipeline_parallel_virtual_stages: int = 1
    pipeline_parallel_input_weight: int = 1
    pipeline_parallel_output_weight: int = 1
    pipeline_parallel_num_layers_in_first_stage: Optional[int] = None
    pipeline_parallel_num_layers_in_last_stage: Optional[int] = None
    pp_seq_len_bucket_size: int = 1024
    pp_variable_seq_lengths: bool = True
    reshard_after_forward: Optional[bool] = None
    cp_fsdp_mode: str = "all"
    fsdp_sharded_lm_head_loss: bool = False
    fsdp_sharded_lm_head_loss_num_chunks: int = 8
    moe_grad_reduce_mode: Literal["reduce_scatter", "bf16_a2a_fp32_sum"] = "reduce_scatter"
    ckpt_manager: Literal["dcp"] = "dcp"
    save_async: bool = False
    load_checkpoint_path: Optional[str] = None
    load_optimizer: bool = True
    save_steps: int = 0
    save_epochs: float = 1
    save_hf_weights: bool = True
    seed: int = 42
    enable_compile: bool = False
    compile_dynamic_shapes: bool = False
    log_format: Literal["progress_bar", "structured", "plain"] = "progress_bar"
    enable_step_phase_timing: bool = False
    step_phase_timing_sync_cuda: bool = True
    enable_per_component_timing: bool = False
    enable_step_memory_profiling: bool = False
    use_wandb: bool = True
    wandb_project: str = "Xorl"
    wandb_name: Optional[str] = None
    wandb_tags: Optional[List[str]] = None
    repo_commit: Optional[str] = None
    wandb_log_interval: int = 1
    enable_profiling: bool = False
    profile_start_step: int = 1
    profile_end_step: int = 2
    profile_trace_dir: str = "./trace"
    profile_record_shapes: bool = True
    profile_profile_memory: bool = True
    profile_with_stack: bool = True
    profile_rank0_only: bool = True
    max_steps: Optional[int] = None
    # ---- keys of this framework (not in the reference) -------------------------------------
    # device / backend for the CPU (gloo) lane; "auto" = cuda+nccl when a GPU is visible
    device: Literal["auto", "cuda", "cpu"] = "auto"
    # per fused communication path: "fused" = own peer-memory kernels, "nccl" = library collectives
    comm_backend: Literal["auto", "fused", "nccl"] = "auto"

    def __post_init__(self):
        if self.ep_outside is not None:
            self.ep_intranode = not self.ep_outside
        if self.moe_checkpoint_method is not None:
            if self.moe_checkpoint_method != "moe_act":
                raise ValueError(f"Unknown moe_checkpoint_method: {self.moe_checkpoint_method!r}")
            if self.gradient_checkpointing_method not in (None, "recompute_before_dispatch"):
                raise ValueError("moe_checkpoint_method='moe_act' conflicts with "
                                 f"gradient_checkpointing_method={self.gradient_checkpointing_method!r}")
            self.gradient_checkpointing_method = "recompute_before_dispatch"
        gcm = self.gradient_checkpointing_method or "recompute_full_layer"
        if gcm not in ("recompute_full_layer", "recompute_before_dispatch", "no_recompute", "moe_act"):
            raise ValueError(f"Unknown gradient_checkpointing_method: {gcm!r}")
        self.gradient_checkpointing_method = gcm
        if self.enable_per_component_timing and not self.enable_step_phase_timing:
            raise ValueError("enable_per_component_timing requires enable_step_phase_timing=True")
        if self.enable_step_memory_profiling and not self.enable_step_phase_timing:
            raise ValueError("enable_step_memory_profiling requires enable_step_phase_timing=True")
        if self.enable_qarl and self.enable_fp8_training:
            raise ValueError("enable_qarl cannot be combined with enable_fp8_training")
        if self.enable_qarl:
            if self.qarl_calib_size < 0:
                raise ValueError("qarl_calib_size must be non-negative")
            if self.qarl_quant_sequence_length is not None and self.qarl_quant_sequence_length <= 0:
                raise ValueError("qarl_quant_sequence_length must be positive when set")
            if self.qarl_calib_data is None and (self.qarl_calib_size or self.qarl_quant_sequence_length is not None):
                raise ValueError("qarl_calib_size and qarl_quant_sequence_length require qarl_calib_data")
            from .adapters.qarl import normalize_quant_cfg
            self.qarl_quant_cfg = normalize_quant_cfg(self.qarl_quant_cfg, default_format=self.qarl_sync_format
                                                      if self.qarl_sync_format != "bf16" else "fp8")
        if self.fp8_cfg:
            self.enable_fp8_training = bool(self.fp8_cfg.get("enabled", True)) or self.enable_fp8_training
        sched = self.pipeline_parallel_schedule.lower()
        if sched not in PP_SCHEDULES:
            raise ValueError(f"pipeline_parallel_schedule must be one of {PP_SCHEDULES}, got "
                             f"{self.pipeline_parallel_schedule!r}")
        if self.cp_fsdp_mode not in ("all", "ulysses_only", "ring_only", "none"):
            raise ValueError(f"cp_fsdp_mode must be all|ulysses_only|ring_only|none, got {self.cp_fsdp_mode!r}")
        if self.micro_batch_size < 1 or self.gradient_accumulation_steps < 1:
            raise ValueError("micro_batch_size and gradient_accumulation_steps must be >= 1")
        if self.lm_head_tensor_parallel_size > 1 and self.tensor_parallel_size > 1:
            raise ValueError("lm_head_tensor_parallel_size > 1 requires tensor_parallel_size == 1")
        if self.data_parallel_mode == "fsdp2" and self.init_device == "cpu" and self.device == "cuda":
            raise ValueError("fsdp2 requires init_device cuda or meta on GPU")
        if os.environ.get("CUDA_LAUNCH_BLOCKING") == "1" and not self.allow_cuda_launch_blocking:
            raise ValueError("CUDA_LAUNCH_BLOCKING=1 serialises every kernel; set "
                             "train.allow_cuda_launch_blocking=true to run anyway")
        self.world_size = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self._derive_parallel_sizes()
        self.checkpoint_dir = os.path.join(self.output_dir, "checkpoints")

    # derived data-parallel sizes (src/xorl/arguments.py:1704-1753)
    def _derive_parallel_sizes(self) -> None:
        ws = self.world_size
        non_dp = (self.pipeline_parallel_size * self.tensor_parallel_size
                  * self.ulysses_parallel_size * self.ringattn_parallel_size)
        if non_dp < 1 or ws % non_dp != 0:
            raise ValueError(f"world size {ws} is not divisible by pp*tp*ulysses*ring = {non_dp}")
        self.data_parallel_size = ws // non_dp
        dp = self.data_parallel_size
        rep, shard = self.data_parallel_replicate_size, self.data_parallel_shard_size
        if self.data_parallel_mode != "fsdp2":
            rep, shard = dp, 1
        elif rep > 0 and shard > 0:
            if rep * shard != dp:
                raise ValueError(f"data_parallel_replicate_size ({rep}) * data_parallel_shard_size "
                                 f"({shard}) != data parallel size ({dp})")
        elif rep > 0:
            if dp % rep:
                raise ValueError(f"data parallel size {dp} not divisible by replicate size {rep}")
            shard = dp // rep
        elif shard > 0:
            if dp % shard:
                raise ValueError(f"data parallel size {dp} not divisible by shard size {shard}")
            rep = dp // shard
        else:
            rep, shard = 1, dp
        self.data_parallel_replicate_size, self.data_parallel_shard_size = rep, shard
        ranks_per_stage = ws // self.pipeline_parallel_size
        if self.expert_parallel_size > 1:
            if self.tensor_parallel_size > 1:
                # tokens are replicated over a tensor-parallel group, so its ranks would dispatch
                # every token once each and the experts would see it tp times
                raise NotImplementedError("expert_parallel_size > 1 with tensor_parallel_size > 1 is not "
                                          "supported: shard the experts (EP) or the dense layers (TP)")
            if ranks_per_stage % self.expert_parallel_size:
                raise ValueError(f"ranks per PP stage ({ranks_per_stage}) not divisible by "
                                 f"expert_parallel_size ({self.expert_parallel_size})")
        self.ep_fsdp_size = ranks_per_stage // max(1, self.expert_parallel_size)
        self.global_batch_size = (self.micro_batch_size * self.gradient_accumulation_steps
                                  * self.data_parallel_size)


@dataclass
class LoRAArguments:
    enable_lora: bool = False
    lora_rank: int = 16
    lora_alpha: int = 16
    lora_b_init_std: float = 0.0
    lora_b_init_seed: int = 0
    lora_target_modules: Optional[List[str]] = None
    lora_target_manifest: Optional[Union[str, Dict[str, Any]]] = None
    unfuse_for_lora: bool = False
    save_lora_only: bool = False
    enable_qlora: bool = False
    block_fp8_qlora_training: bool = False
    quant_format: str = "nvfp4"
    quant_group_size: int = 16
    merge_lora_interval: int = 0
    reset_optimizer_on_merge: bool = False
    exclude_modules: Optional[List[str]] = None
    enable_aqn: bool = False
    aqn_alpha: float = 1.0
    moe_hybrid_shared_lora: bool = False

    def __post_init__(self):
        if self.enable_qlora:
            self.enable_lora = True
        if self.quant_format not in ("nvfp4", "block_fp8", "nf4", "int4", "mxfp4"):
            raise ValueError(f"unknown quant_format {self.quant_format!r}")
        if self.lora_rank < 1:
            raise ValueError("lora_rank must be >= 1")


@dataclass
class DistillationArguments:
    enable_distillation: bool = False
    teacher_model_path: Optional[str] = None
    distillation_loss_type: str = "forward_kl"
    distillation_loss_weight: float = 1.0
    stream_num_workers: int = 32


@dataclass
class Arguments:
    model: ModelArguments = field(default_factory=ModelArguments)
    data: DataArguments = field(default_factory=DataArguments)
    train: TrainingArguments = field(default_factory=TrainingArguments)
    distill: DistillationArguments = field(default_factory=DistillationArguments)
    lora: LoRAArguments = field(default_factory=LoRAArguments)

    def __post_init__(self):
        t = self.train
        if t.tensor_parallel_size > 1 and self.lora.enable_lora:
            raise ValueError("tensor parallelism cannot be combined with LoRA")
        if t.pipeline_parallel_size > 1 and self.data.sample_packing_sequence_len is None:
            raise ValueError("pipeline parallelism requires sample packing")
        if t.enable_qarl and (self.lora.enable_lora or self.lora.enable_qlora):
            raise ValueError("enable_qarl trains the full weights and cannot be combined with LoRA or QLoRA")
        # keys whose value asks for something that is not built raise here instead of being ignored
        from .config_policy import check_supported
        for section in ("model", "data", "train", "lora", "distill"):
            check_supported(section, getattr(self, section))


# ------------------------------------------------------------------------------------------------
# parsing
# ------------------------------------------------------------------------------------------------
def _strip_optional(tp):
    origin = get_origin(tp)
    if origin is Union or (hasattr(types, "UnionType") and isinstance(tp, types.UnionType)):
        args = [a for a in get_args(tp) if a is not type(None)]
        if len(args) == 1:
            return args[0], True
        return tp, True
    return tp, False


def _convert(value: Any, tp: Any, name: str) -> Any:
    """Converts a CLI string (or YAML scalar) to the declared field type."""
    tp, optional = _strip_optional(tp)
    if value is None:
        return None
    if isinstance(value, str) and optional and value.lower() in ("none", "null"):
        return None
    origin = get_origin(tp)
    if origin is Literal:
        choices = get_args(tp)
        for c in choices:
            if value == c or (isinstance(value, str) and str(c) == value):
                return c
        raise ValueError(f"{name}: {value!r} is not one of {choices}")
    if tp is bool:
        if isinstance(value, bool):
            return value
        if isinstance(value, str):
            if value.lower() in ("1", "true", "yes", "y", "t"):
                return True
            if value.lower() in ("0", "false", "no", "n", "f"):
                return False
        raise ValueError(f"{name}: cannot interpret {value!r} as bool")
    if tp is int:
        if isinstance(value, bool):
            raise ValueError(f"{name}: expected int, got bool")
        return int(value)
    if tp is float:
        return float(value)
    if tp is str:
        return str(value)
    if origin in (list, List, dict, Dict) or tp in (list, dict) or origin is Union:
        if isinstance(value, str):
            try:
                return json.loads(value)
            except json.JSONDecodeError:
                if origin in (list, List) or tp is list:
                    return [v for v in value.split(",") if v]
                if origin is Union:
                    return value
                raise ValueError(f"{name}: expected JSON for {tp}, got {value!r}")
        return value
    return value


def _load_file(path: str) -> Dict[str, Any]:
    with open(path) as f:
        if path.endswith(".json"):
            return json.load(f) or {}
        return yaml.safe_load(f) or {}


def parse_args(rootclass=Arguments, argv: Optional[List[str]] = None):
    """``prog cfg.yaml --train.lr 1e-4 --model.merge_qkv=false``; CLI overrides YAML; unknown keys
    raise ValueError."""
    argv = list(sys.argv[1:] if argv is None else argv)
    file_cfg: Dict[str, Any] = {}
    if argv and not argv[0].startswith("--"):
        file_cfg = _load_file(argv.pop(0))
    # NeMo-style fp8 block compat: `train.fp8: {enabled: true, ...}` -> fp8_cfg
    if isinstance(file_cfg.get("train"), dict) and "fp8" in file_cfg["train"]:
        file_cfg["train"]["fp8_cfg"] = file_cfg["train"].pop("fp8")

    cli: Dict[str, Dict[str, Any]] = {}
    i = 0
    while i < len(argv):
        tok = argv[i]
        if not tok.startswith("--"):
            raise ValueError(f"unexpected argument {tok!r}")
        key = tok[2:]
        if "=" in key:
            key, val = key.split("=", 1)
            i += 1
        elif i + 1 < len(argv) and not argv[i + 1].startswith("--"):
            val = argv[i + 1]
            i += 2
        else:
            val = "true"  # bare boolean flag
            i += 1
        if "." not in key:
            raise ValueError(f"override {tok!r} must be of the form --section.field")
        sec, name = key.split(".", 1)
        cli.setdefault(sec, {})[name] = val

    return build_args(file_cfg, cli, rootclass)


def build_args(file_cfg: Dict[str, Any], cli: Optional[Dict[str, Dict[str, Any]]] = None, rootclass=Arguments):
    """Arguments from a nested ``{section: {key: value}}`` mapping (plus optional overrides)."""
    cli = cli or {}
    sections = {f.name: f.default_factory for f in fields(rootclass)}
    unknown = [s for s in list(file_cfg) + list(cli) if s not in sections]
    if unknown:
        raise ValueError(f"unknown config section(s): {sorted(set(unknown))}")

    built = {}
    for sec, cls in sections.items():
        hints = get_type_hints(cls)
        valid = {f.name for f in fields(cls) if f.init}
        merged: Dict[str, Any] = {}
        for src in (file_cfg.get(sec) or {}, cli.get(sec) or {}):
            for k, v in src.items():
                if k not in valid:
                    raise ValueError(f"unknown config key {sec}.{k}")
                merged[k] = _convert(v, hints[k], f"{sec}.{k}")
        built[sec] = cls(**merged)
    return rootclass(**built)


def _plain(obj: Any) -> Any:
    if is_dataclass(obj):
        return {f.name: _plain(getattr(obj, f.name)) for f in fields(obj) if f.init}
    if isinstance(obj, dict):
        return {k: _plain(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [_plain(v) for v in obj]
    return obj


def save_args(args, output_dir: str) -> str:
    """Writes the resolved configuration to ``{output_dir}/xorl_cli.yaml``."""
    os.makedirs(output_dir, exist_ok=True)
    path = os.path.join(output_dir, "xorl_cli.yaml")
    with open(path, "w") as f:
        yaml.safe_dump(_plain(args), f, sort_keys=False)
    return path
