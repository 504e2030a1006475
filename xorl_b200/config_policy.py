"""What happens to a configuration key that no code path reads.

The YAML schema mirrors the reference's (src/xorl/arguments.py) field for field so that its
configurations load unchanged.  A key falls into exactly one class:

* it is read somewhere in the package (``tests/test_cli_cpu.py`` finds the reader by text search);
* ``SATISFIED_BY_DESIGN``: every value it can take asks for something this framework always does,
  or selects among alternatives of which this framework has exactly one (for instance the
  reference's choice between a Triton, a compiled and a "native" RMSNorm: there is one kernel here).
  Such keys are accepted as they are; the entry says why nothing needs to change;
* ``UNSUPPORTED``: some values ask for behaviour that is not built.  The entry lists the values that
  are accepted; any other value raises ``NotImplementedError`` naming the key
  (``check_supported``), instead of being silently ignored.
"""
from __future__ import annotations

from typing import Any, Callable, Dict, Tuple

# section -> key -> reason
SATISFIED_BY_DESIGN: Dict[str, Dict[str, str]] = {
    "model": {
        "moe_routing_weights_before_down": "a rounding-point choice of the reference's Triton expert backend (same "
                                           "mathematics); here the routing weights are applied in fp32 by the combine",
        "flash_attention_deterministic": "the attention backward has no atomics: it is deterministic with either value",
        "merge_qkv": "projections are always fused in memory; checkpoint handlers split and merge on disk",
        "rmsnorm_mode": "one RMSNorm kernel (csrc/norm.cu); the reference's implementation families do not exist here",
        "qwen35_rmsnorm_family": "same: a single zero-centred RMSNorm implementation",
        "activation_native": "one SwiGLU kernel with the two-round rounding of the reference's native path",
        "rope_native": "one rotary implementation (fused with qk-norm, fp32 math)",
        "rope_class_b": "same: rotary math is always fp32 inside the kernel",
        "attention_cast_bf16": "attention operands are bf16 in the only attention kernel",
        "deepep_buffer_size_gb": "DeepEP is replaced by the peer-memory path, which sizes its own workspace",
        "deepep_num_sms": "same: the push kernels use a fixed small grid",
        "deepep_async_combine": "same: dispatch and combine are stream-ordered kernels without a host-visible handle",
        "alltoall_combine_hidden_chunk_size": "the all-to-all combine is not chunked; results are identical",
        "basic_modules": "ZeRO units are built per decoder layer from the model itself",
        "encoders": "multi-modal encoders are outside the text-only model families of this package",
        "record_routing_weights": "routing weights are recomputed from the recorded expert choices when a layer is replayed",
    },
    "data": {
        "dataloader_num_workers": "the packed loader prefetches on a background thread; worker processes are not needed",
        "sample_packing_bin_size": "the C++ packer processes a whole group (sample_packing_group_size) at once",
        "sample_packing_sequentially": "chosen by sample_packing_method",
        "sample_packing_mp_start_method": "packing runs in-process in C++",
        "dataset_num_proc": "tokenised datasets are prepared in a single process",
        "shuffle_before_merging_datasets": "datasets are shuffled once after merging (shuffle_merged_datasets)",
        "skip_prepare_dataset": "preparation is lazy and cached; there is no separate step to skip",
        "is_preprocess": "set by the preprocess CLI for itself",
        "fa_max_length_bucket": "the attention kernel takes cu_seqlens directly and needs no max-length buckets",
        "hf_use_auth_token": "no network access is ever attempted",
    },
    "train": {
        "enable_reentrant": "recomputation is done by the engine, not by torch.utils.checkpoint",
        "fp8_training_moe_grouped_backend": "the grouped fp8 expert GEMM has one backend here, the tcgen05 block-scaled "
                                            "kernel (csrc/grouped_gemm_mx.cu), whichever of the reference's is named",
        "muon_distributed_mode": "Newton-Schulz always runs on the whole matrix (the update direction is gathered over "
                                 "the shard group and each rank keeps its slice of the result): the exact form, "
                                 "full_gradient; there is no approximate shard-local mode",
        "prewarm_cuda_blas": "no cuBLAS handle exists on the product path",
        "pp_variable_seq_lengths": "the pipeline runner always negotiates per-micro-batch sequence lengths",
        "pp_seq_len_bucket_size": "stage-to-stage buffers are allocated per micro-batch, not per bucket",
        "ckpt_manager": "DCP is the only checkpoint manager (the only value of the reference's Literal)",
        "repo_commit": "informational; written back with the saved arguments",
        "muon_ns_use_quack_kernels": "Newton-Schulz runs on this package's own GEMM kernels",
        "muon_grouped_gram_ns_fp32_byte_limit": "Gram matrices are formed per parameter, never batched beyond memory",
        "skip_param_upcast": "master weights are fp32 shards by construction",
        "high_precision_bf16": "accumulation is fp32 in every kernel",
        "compile_dynamic_shapes": "only meaningful with enable_compile",
        "fp8_training_blackwell_validation_artifact": "informational path recorded by the reference's guard",
        "fp8_training_allow_bf16_fallback": "operands that cannot be quantised raise instead of falling back",
        "defer_grad_sync_in_accumulation": "replica all-reduces always run once per step, after the last micro-batch",
        "enable_full_shard": "ZeRO-3 sharding of parameters, gradients and optimizer state is the engine's only sharded mode",
        "activation_gpu_limit": "activation offload moves every saved layer input; there is no partial budget",
        "activation_offload_prefetch_count": "the offloader prefetches one layer ahead",
        "log_format": "step metrics are logged as one line per step and to metrics.jsonl / wandb",
        "ce_mode": "one fused lm-head + cross-entropy kernel path",
    },
    "lora": {
        "unfuse_for_lora": "fused projections carry one adapter per output slice (q / k / v, gate / up) with the "
                           "same mathematics as adapters on unfused projections, so nothing needs to be split",
    },
    "distill": {
        "stream_num_workers": "teacher scores are produced in-process, one forward pass per micro-batch",
    },
}


def _is(*allowed) -> Callable[[Any], bool]:
    return lambda v: v in allowed


def _falsy(v) -> bool:
    return not v


# section -> key -> (predicate on the value: True = supported, what is missing)
UNSUPPORTED: Dict[str, Dict[str, Tuple[Callable[[Any], bool], str]]] = {
    "model": {
        "sparse_mla_enabled": (_falsy, "sparse MLA kernels are not built; attention over selected keys runs as masked softmax"),
        "sparse_mla_backend": (_is("auto"), "no selectable sparse-MLA backend"),
    },
    "data": {
        "push_dataset_to_hub": (_falsy, "no network access"),
    },
    "train": {
        "anyprecision_adamw_reuse_grad_for_momentum": (_falsy, "the optimizer step never writes the gradient shard (other streams order "
                                                                "themselves against reads of it only)"),
        "muon_fallback_optimizer": (_is("adamw"), "non-matrix parameters under Muon always use AdamW"),
        "muon_grad_dtype": (_falsy, "Muon works on the fp32 gradient shards"),
        "muon_update_dtype": (_falsy, "Muon updates are bf16 Newton-Schulz iterates applied to fp32 masters"),
        "muon_force_momentum_path": (_falsy, "not built"),
        "fp8_training_block_size": (_is(128), "block fp8 uses 128-wide blocks (1 x 128 activations, 128 x 128 weights)"),
        "fp8_training_smoothquant_alpha": (_falsy, "SmoothQuant rescaling is not built"),
        "fp8_training_lm_head_smoothquant_alpha": (_falsy, "SmoothQuant rescaling is not built"),
        "fp8_training_activation_amax_scale": (_is(1.0, 1), "amax margins are not built"),
        "fp8_training_weight_amax_scale": (_is(1.0, 1), "amax margins are not built"),
        "fp8_training_correction_mode": (_is("none"), "residual correction is not built"),
        "enable_compile": (_falsy, "there is no tracing compiler on any path"),
    },
    "lora": {
        "block_fp8_qlora_training": (_falsy, "fp8 training of QLoRA bases is not built"),
    },
}


def check_supported(section: str, obj) -> None:
    """Raises NotImplementedError for the first key of ``section`` whose value asks for something
    that is not built."""
    for key, (ok, why) in UNSUPPORTED.get(section, {}).items():
        if not hasattr(obj, key):
            continue
        v = getattr(obj, key)
        if not ok(v):
            raise NotImplementedError(f"{section}.{key}={v!r} is not supported: {why}")
