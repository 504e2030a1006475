"""Flat configuration of the training service and its translation into the trainer's sectioned
arguments (src/xorl/server/server_arguments.py).  One YAML level: model, parallelism, optimizer
family, packing and service knobs side by side."""
from __future__ import annotations

from dataclasses import dataclass, field, fields
from typing import Any, Dict, List, Optional

import yaml

from ..arguments import Arguments, build_args


@dataclass
class ServerArguments:
    # model
    model_path: Optional[str] = None
    config_path: Optional[str] = None
    model_preset: Optional[str] = None
    attn_implementation: str = "native"
    moe_implementation: str = "native"
    # parallelism
    data_parallel_mode: str = "fsdp2"
    data_parallel_shard_size: int = -1
    data_parallel_replicate_size: int = 1
    tensor_parallel_size: int = 1
    pipeline_parallel_size: int = 1
    ulysses_parallel_size: int = 1
    ringattn_parallel_size: int = 1
    expert_parallel_size: int = 1
    # training
    optimizer: str = "adamw"
    weight_decay: float = 0.0
    enable_mixed_precision: bool = True
    enable_gradient_checkpointing: bool = True
    seed: int = 42
    output_dir: str = "outputs/server"
    device: str = "auto"
    comm_backend: str = "auto"
    # adapters
    enable_lora: bool = False
    lora_rank: int = 16
    lora_alpha: int = 32
    lora_target_modules: Optional[List[str]] = None
    enable_qlora: bool = False
    quant_format: str = "nvfp4"
    max_adapters_per_model: int = 8
    # quantisation-aware RL: full-weight training on the grid the inference engine serves
    enable_qarl: bool = False
    qarl_quant_cfg: Optional[Any] = None
    qarl_calib_data: Optional[str] = None
    qarl_calib_size: int = 0
    qarl_quant_sequence_length: Optional[int] = None
    qarl_sync_format: str = "fp8"
    qarl_target_modules: Optional[List[str]] = None
    qarl_exclude_modules: Optional[List[str]] = None
    # service
    api_host: str = "127.0.0.1"
    api_port: int = 8000
    sample_packing_sequence_len: int = 4096
    sample_packing_method: str = "sequential"           # sequential | best_fit | balanced_dp
    sample_packing_strategy: Optional[str] = None        # the reference's newer name; wins when set
    sample_packing_on_oversized: str = "error"           # error | skip | truncate
    future_ttl_seconds: float = 3600.0
    session_timeout_seconds: float = 600.0
    idle_sleep_seconds: float = 0.0
    api_keys: List[str] = field(default_factory=list)
    worker_bind_address: str = "tcp://127.0.0.1:5555"
    sync_bucket_size_mb: int = 1024
    storage_limit_gb: float = 0.0                        # saves are refused (507) beyond this much under output_dir; 0 = no limit
    enable_moe_metrics: bool = True                      # moe_metrics.jsonl for MoE models

    def __post_init__(self) -> None:
        """Cross-field checks that would otherwise surface deep inside the worker fleet
        (src/xorl/server/server_arguments.py:1230-1260)."""
        strategy = self.sample_packing_strategy or self.sample_packing_method
        if strategy not in ("sequential", "best_fit", "balanced_dp"):
            raise ValueError(f"sample_packing_strategy must be sequential, best_fit or balanced_dp, got {strategy!r}")
        if self.sample_packing_on_oversized not in ("error", "skip", "truncate"):
            raise ValueError("sample_packing_on_oversized must be error, skip or truncate, "
                             f"got {self.sample_packing_on_oversized!r}")
        if self.sample_packing_sequence_len < 1:
            raise ValueError("sample_packing_sequence_len must be positive")
        for name in ("tensor_parallel_size", "pipeline_parallel_size", "ulysses_parallel_size",
                     "ringattn_parallel_size", "expert_parallel_size", "data_parallel_replicate_size"):
            if getattr(self, name) < 1:
                raise ValueError(f"{name} must be at least 1")
        if not (0 < int(self.api_port) < 65536):
            raise ValueError(f"api_port {self.api_port} is not a TCP port")
        if self.enable_qlora and not self.enable_lora:
            raise ValueError("enable_qlora needs enable_lora (the quantised base is frozen; only adapters train)")
        if self.enable_qarl and (self.enable_lora or self.enable_qlora):
            raise ValueError("enable_qarl trains the full weights and cannot be combined with LoRA or QLoRA")
        if self.max_adapters_per_model < 1:
            raise ValueError("max_adapters_per_model must be at least 1")
        if self.future_ttl_seconds <= 0 or self.session_timeout_seconds <= 0:
            raise ValueError("future_ttl_seconds and session_timeout_seconds must be positive")
        if not self.worker_bind_address.startswith(("tcp://", "ipc://")):
            raise ValueError(f"worker_bind_address must be a tcp:// or ipc:// ZMQ address, got {self.worker_bind_address!r}")

    @classmethod
    def from_yaml(cls, path: str, overrides: Optional[Dict[str, Any]] = None) -> "ServerArguments":
        with open(path) as f:
            raw = yaml.safe_load(f) or {}
        raw.update(overrides or {})
        known = {f.name for f in fields(cls)}
        unknown = sorted(set(raw) - known)
        if unknown:
            raise ValueError(f"unknown server config keys: {unknown}")
        return cls(**raw)

    def to_trainer_arguments(self) -> Arguments:
        """Sectioned arguments for the in-process trainer the runner is built on."""
        d = {
            "model": {"model_path": self.model_path, "config_path": self.config_path,
                      "attn_implementation": self.attn_implementation,
                      "moe_implementation": self.moe_implementation},
            "data": {"datasets": [{"type": "dummy", "path": "dummy"}],
                     "sample_packing_sequence_len": self.sample_packing_sequence_len},
            "train": {"output_dir": self.output_dir, "optimizer": self.optimizer,
                      "weight_decay": self.weight_decay, "seed": self.seed,
                      "data_parallel_mode": self.data_parallel_mode,
                      "data_parallel_shard_size": self.data_parallel_shard_size,
                      "data_parallel_replicate_size": self.data_parallel_replicate_size,
                      "tensor_parallel_size": self.tensor_parallel_size,
                      "pipeline_parallel_size": self.pipeline_parallel_size,
                      "ulysses_parallel_size": self.ulysses_parallel_size,
                      "ringattn_parallel_size": self.ringattn_parallel_size,
                      "expert_parallel_size": self.expert_parallel_size,
                      "enable_mixed_precision": self.enable_mixed_precision,
                      "enable_gradient_checkpointing": self.enable_gradient_checkpointing,
                      "device": self.device, "comm_backend": self.comm_backend,
                      "enable_qarl": self.enable_qarl, "qarl_quant_cfg": self.qarl_quant_cfg,
                      "qarl_calib_data": self.qarl_calib_data, "qarl_calib_size": self.qarl_calib_size,
                      "qarl_quant_sequence_length": self.qarl_quant_sequence_length,
                      "qarl_sync_format": self.qarl_sync_format,
                      "qarl_target_modules": self.qarl_target_modules,
                      "qarl_exclude_modules": self.qarl_exclude_modules,
                      "max_steps": 1, "lr_warmup_ratio": 0.0, "lr_decay_style": "constant"},
            "lora": {"enable_lora": self.enable_lora, "lora_rank": self.lora_rank,
                     "lora_alpha": self.lora_alpha, "lora_target_modules": self.lora_target_modules,
                     "enable_qlora": self.enable_qlora, "quant_format": self.quant_format},
        }
        if self.model_preset and not (self.model_path or self.config_path):
            d["model"]["config_path"] = self.model_preset
        return build_args(d)
