"""Reference arm of bench.py: runs the UNMODIFIED reference (installed under ``baseline/_ref``)
through its own public API — ``xorl.arguments.parse_args`` -> ``xorl.trainers.trainer.Trainer`` ->
``Trainer.train_step`` — on the same metric and configuration as our arm: Qwen3-8B, bf16, FSDP2,
seq 4096, micro-batch 1 per GPU, packed documents with lengths U[256, 4096], AdamW, activations
kept (``gradient_checkpointing_method: no_recompute``, the faster setting for both arms; ``--recompute
full`` turns recomputation on in both), random-init weights.  None of this repository's models, kernels or engine is
imported on this path.

Offline constraints recorded here: the reference's FlashAttention-3/4 wheels are not installed in
this image, so its attention runs through its ``native`` (torch SDPA) backend, which is the stock
path it offers without those wheels.
"""
from __future__ import annotations

import json
import os
import socket
import sys
import time

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

QWEN3_8B = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "vocab_size": 151936,
    "hidden_size": 4096, "intermediate_size": 12288, "num_hidden_layers": 36,
    "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128, "hidden_act": "silu",
    "max_position_embeddings": 40960, "rms_norm_eps": 1e-6, "rope_theta": 1000000.0,
    "rope_scaling": None, "tie_word_embeddings": False, "attention_bias": False,
    "attention_dropout": 0.0, "initializer_range": 0.02, "torch_dtype": "bfloat16",
    "use_cache": False, "sliding_window": None, "use_sliding_window": False,
    "max_window_layers": 36, "bos_token_id": 151643, "eos_token_id": 151645,
}


QWEN3_30B_A3B = {
    "architectures": ["Qwen3MoeForCausalLM"], "model_type": "qwen3_moe", "vocab_size": 151936,
    "hidden_size": 2048, "intermediate_size": 6144, "moe_intermediate_size": 768,
    "num_hidden_layers": 48, "num_attention_heads": 32, "num_key_value_heads": 4, "head_dim": 128,
    "num_experts": 128, "num_experts_per_tok": 8, "norm_topk_prob": True, "decoder_sparse_step": 1,
    "mlp_only_layers": [], "output_router_logits": True, "router_aux_loss_coef": 0.001,
    "hidden_act": "silu", "max_position_embeddings": 40960, "rms_norm_eps": 1e-6,
    "rope_theta": 1000000.0, "rope_scaling": None, "tie_word_embeddings": False,
    "attention_bias": False, "attention_dropout": 0.0, "initializer_range": 0.02,
    "torch_dtype": "bfloat16", "use_cache": False, "sliding_window": None,
    "use_sliding_window": False, "max_window_layers": 48, "bos_token_id": 151643,
    "eos_token_id": 151645,
}
MODELS = {"qwen3-8b": QWEN3_8B, "qwen3-30b-a3b": QWEN3_30B_A3B}


def _unavailable(why: str) -> None:
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)


def _recompute_method(choice: str, world: int) -> str:
    """The reference's own ``train.gradient_checkpointing_method`` values.  ``auto`` keeps the
    activations (no recomputation) when the sharded state leaves room for them, as our arm does."""
    if choice == "full":
        return "recompute_full_layer"
    if choice == "none":
        return "no_recompute"
    # measured on one B200: the reference holds Qwen3-8B's activations beside the unsharded state
    # (691 ms/step against 756 ms with recomputation), so fewer parameters per rank fit as well
    return "no_recompute"


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _write_model_dir(path: str, layers: int = 0, model: str = "qwen3-8b") -> None:
    """config.json of the named architecture plus a minimal local tokenizer (the dummy dataset is
    pre-tokenised; the reference only asks the tokenizer for its length and special ids)."""
    os.makedirs(path, exist_ok=True)
    cfg = dict(MODELS[model])
    if layers:
        cfg["num_hidden_layers"] = layers
        cfg["max_window_layers"] = layers
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast
    vocab = {f"t{i}": i for i in range(4094)}
    vocab["<pad>"] = 4094
    vocab["<eos>"] = 4095
    tok = Tokenizer(models.WordLevel(vocab, unk_token="t0"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, pad_token="<pad>", eos_token="<eos>",
                                   unk_token="t0")
    fast.save_pretrained(path)


def _yaml(model_dir: str, out_dir: str, seq_len: int, world: int, gcm: str, moe: bool = False,
          ep: int = 1) -> str:
    # MoE: the reference's stock expert backend (Triton grouped GEMM) and dispatch (all-to-all) that
    # import offline; bf16 experts, since it refuses fp8 training on this architecture
    # (src/xorl/fp8_training/config_compat.py:293-306)
    moe_model = "  moe_implementation: triton\n  ep_dispatch: alltoall\n" if moe else ""
    moe_train = f"  expert_parallel_size: {ep}\n" if moe else ""
    return f"""
model:
  config_path: {model_dir}
  tokenizer_path: {model_dir}
  attn_implementation: native
{moe_model}data:
  datasets:
    - path: dummy
      type: tokenized
      max_seq_len: {seq_len}
      num_samples: {max(64, 8 * world)}
  select_columns: [input_ids, labels]
  sample_packing_method: sequential
  sample_packing_sequence_len: {seq_len}
  dataloader_num_workers: 0
  dataloader_pin_memory: true
train:
  output_dir: {out_dir}
  data_parallel_mode: fsdp2
  data_parallel_replicate_size: 1
  data_parallel_shard_size: {world}
{moe_train}  micro_batch_size: 1
  gradient_accumulation_steps: 1
  optimizer: adamw
  lr: 1.0e-5
  weight_decay: 0.01
  max_grad_norm: 1.0
  enable_mixed_precision: true
  enable_gradient_checkpointing: true
  gradient_checkpointing_method: {gcm}
  init_device: meta
  num_train_epochs: 1000
  max_steps: 1000000
  save_steps: 0
  save_epochs: 0
  save_hf_weights: false
  use_wandb: false
  log_format: structured
"""


def run_reference(a) -> None:
    if not os.path.isdir(os.path.join(REF, "xorl")):
        _unavailable("baseline/_ref is empty: the reference is not installed on this machine")
        return
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(_free_port()))
    os.environ.setdefault("WANDB_MODE", "disabled")
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ.setdefault("TOKENIZERS_PARALLELISM", "false")
    world, rank = int(os.environ["WORLD_SIZE"]), int(os.environ["RANK"])
    # the reference must be importable as `xorl`; this repository's own package must not be used
    sys.path = [p for p in sys.path if os.path.abspath(p or ".") != ROOT]
    sys.path.insert(0, REF)
    scratch = getattr(a, "scratch_dir", "") or os.path.join(__import__("tempfile").gettempdir(), "xorl_b200_bench")
    work = os.path.join(scratch, "ref_run")
    gcm = _recompute_method(getattr(a, "recompute", "auto"), world)
    model = getattr(a, "model", "qwen3-8b")
    if model not in MODELS:
        _unavailable(f"the reference arm has no configuration for model {model!r}")
        return
    moe = model == "qwen3-30b-a3b"
    ep = (getattr(a, "ep", 0) or world) if moe else 1
    if moe and gcm == "no_recompute" and getattr(a, "recompute", "auto") == "auto":
        gcm = "recompute_full_layer"          # same setting as our arm for the MoE model
    model_dir = os.path.join(work, model.replace("-", "_"))
    # named after this launch's rendezvous port, so ranks never pick up an earlier run's file
    cfg_path = os.path.join(work, f"cfg_{os.environ['MASTER_PORT']}_{gcm}.yaml")
    try:
        if rank == 0:
            _write_model_dir(model_dir, getattr(a, "layers", 0), model)
            with open(cfg_path, "w") as f:
                f.write(_yaml(model_dir, os.path.join(work, "out"), a.seq_len, world, gcm, moe, ep))
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
        # wait for rank 0's files without a collective (the reference initialises the process group)
        for _ in range(600):
            if os.path.exists(cfg_path):
                break
            time.sleep(0.1)
        time.sleep(0.5 if rank else 0.0)
        sys.argv = ["xorl.cli.train", cfg_path]
        from xorl.arguments import Arguments, parse_args
        from xorl.trainers.trainer import Trainer
        args = parse_args(Arguments)
        trainer = Trainer(args)
        _measure(trainer, a, world, rank, model, ep)
    except Exception as e:  # noqa: BLE001
        import traceback
        traceback.print_exc()
        _unavailable(f"reference failed to run here: {type(e).__name__}: {str(e)[:300]}")


def _synthetic_like(example, seq_len: int, vocab: int, seed: int):
    """A micro-batch with the reference collator's keys and shapes, filled with packed documents of
    lengths U[256, seq_len] and uniform tokens (same generator as our arm)."""
    import numpy as np
    import torch
    from xorl.data.collators.packing_concat_collator import add_flash_attention_kwargs_from_position_ids
    rng = np.random.default_rng(seed)
    ids = rng.integers(0, vocab, size=seq_len + 1, dtype=np.int64)
    cu = [0]
    while cu[-1] < seq_len:
        cu.append(min(seq_len, cu[-1] + int(rng.integers(256, seq_len + 1))))
    labels = ids[1:].copy()
    pos = np.zeros(seq_len, dtype=np.int64)
    for s, e in zip(cu[:-1], cu[1:]):
        pos[s:e] = np.arange(e - s)
        labels[e - 1] = -100
    shape = tuple(example["input_ids"].shape)
    batch = {}
    for k, v in example.items():
        if k in ("input_ids", "labels", "position_ids") or k.startswith(("cu_seq_lens", "max_length")):
            continue
        batch[k] = v
    batch["input_ids"] = torch.from_numpy(ids[:-1].copy()).reshape(shape).to(example["input_ids"].dtype)
    batch["labels"] = torch.from_numpy(labels).reshape(shape).to(example["labels"].dtype)
    batch["position_ids"] = torch.from_numpy(pos).reshape(tuple(example["position_ids"].shape)) \
        .to(example["position_ids"].dtype)
    if "attention_mask" in batch:
        batch["attention_mask"] = torch.ones_like(example["attention_mask"])
    if any(k.startswith("cu_seq_lens") for k in example):
        add_flash_attention_kwargs_from_position_ids(batch)
    return {k: (v.pin_memory() if torch.is_tensor(v) and not v.is_cuda else v) for k, v in batch.items()}


def _measure(trainer, a, world: int, rank: int, model: str = "qwen3-8b", ep: int = 1) -> None:
    import torch
    import torch.distributed as dist
    from xorl.distributed.offloading import build_activation_offloading_context
    args = trainer.args
    # the same preamble Trainer.train() runs before its loop
    fwd_ctx, bwd_ctx = build_activation_offloading_context(
        args.train.enable_activation_offload, args.train.enable_gradient_checkpointing,
        args.train.activation_gpu_limit, args.train.activation_offload_prefetch_count)
    trainer._model_fwd_context, trainer._model_bwd_context = fwd_ctx, bwd_ctx
    for part in trainer._all_model_parts():
        part.train()
    example = next(iter(trainer.train_dataloader))[0]
    seq_len = int(example["input_ids"].numel())
    vocab = int(trainer.model_config.vocab_size)
    n_total = a.warmup + a.steps
    batches = [[_synthetic_like(example, seq_len, vocab, 1000 * rank + s)] for s in range(n_total)]
    dev = torch.device("cuda", int(os.environ["LOCAL_RANK"]))

    def barrier():
        if dist.is_initialized() and world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sys.path.insert(0, ROOT)  # only for the clock sampler helper of bench.py (no package import)
    from bench import ClockSampler
    for s in range(a.warmup):
        trainer.train_step(batches[s])
    barrier()
    sampler = ClockSampler(int(os.environ["LOCAL_RANK"]))
    sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    loss = 0.0
    for s in range(a.warmup, n_total):
        loss, _ = trainer.train_step(batches[s])      # host batches: H2D inside, loss read inside
    e1.record()
    barrier()
    wall = time.perf_counter() - t0
    clocks = sampler.stop()
    t = torch.tensor([e0.elapsed_time(e1), wall * 1e3], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = t[0].item() / a.steps
    tokens = seq_len * world
    h2d = sum(v.numel() * v.element_size() for v in batches[0][0].values() if torch.is_tensor(v))
    if rank == 0:
        print(json.dumps({
            "metric": "tokens/sec (device-timed, max over ranks) Qwen3-8B/30B-A3B at 1/2/4/8 B200",
            "value": tokens / (ms_per_step / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "reference",
            "config": {"model": model + (f"[{a.layers} layers: DEBUG]" if getattr(a, "layers", 0) else ""),
                       "global_batch": world, "seq_len": seq_len,
                       "parallelism": f"fsdp{world}" + (f"-ep{ep}-alltoall" if ep > 1 else ""),
                       "attn_implementation": str(args.model.attn_implementation),
                       "recompute": str(args.train.gradient_checkpointing_method),
                       "l2": "per-step working set >> 126 MB L2",
                       "packed_docs": "lengths U[256,4096], tokens U[vocab]"},
            "clocks": clocks,
            "e2e": {"value": tokens * a.steps / (t[1].item() / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": h2d * world, "d2h_bytes_per_step": 4 * world},
            "gpu_launches": 0, "loss": float(loss),
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 2 ** 30}), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
