"""Every parallel mode on real GPUs (bf16, hand-written kernels) against a single-GPU run of the
same model and data: ZeRO-3, TP, PP (two schedules), Ulysses, ring, hybrid CP, EP.

Two checks that a wrong gradient cannot pass:
* the same four packed rows are trained for 20 steps at a learning rate where the single-GPU loss
  falls by more than 1.0, and the parallel run must follow that curve step by step;
* after the first backward the fully reduced gradient of EVERY parameter (gathered to its
  unsharded shape) is compared with the single-GPU gradient.
"""
import glob
import json
import os
import sys

import pytest
import torch
import yaml

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
pytestmark = [pytest.mark.gpu, pytest.mark.distributed]
ENV = {"NCCL_NVLS_ENABLE": "0"}
STEPS = 20


def _cfg(tmp, name, model="small-qwen3", dp=1, foundation=None, **train):
    # 16 samples -> four rows of 2048 tokens; one optimizer step consumes all four (4 / dp micro-batches
    # per rank), so every step of every layout sees the same global batch
    cfg = {
        "model": {"config_path": model, **({"foundation": dict(foundation)} if foundation else {})},
        "data": {"datasets": [{"path": "random", "type": "tokenized", "max_seq_len": 700,
                               "min_seq_len": 400, "num_samples": 16}],
                 "sample_packing_sequence_len": 2048, "pad_to_multiple_of": 128,
                 "shuffle_merged_datasets": False},
        "train": {"output_dir": str(tmp / name), "lr": 1e-3, "max_steps": STEPS, "use_wandb": False,
                  "save_hf_weights": False, "save_epochs": 0, "gradient_accumulation_steps": 4 // dp, "num_train_epochs": 1000,
                  "weight_decay": 0.0, **train},
    }
    p = tmp / f"{name}.yaml"
    p.write_text(yaml.safe_dump(cfg))
    return str(p)


def _losses(tmp, name):
    with open(tmp / name / "training_metrics.json") as f:
        return json.load(f)["loss_history"]


def _grads(tmp, name):
    out = {}
    for f in sorted(glob.glob(str(tmp / name / "grads" / "grads_pp*.pt"))):
        out.update(torch.load(f))
    return out


def _run(tmp, name, nproc, model="small-qwen3", dp=1, extra_cli=(), foundation=None, **train):
    from dist_utils import run_distributed
    env = dict(ENV, XORL_DEBUG_DUMP_GRADS=str(tmp / name / "grads"))
    run_distributed("-m", nproc, "xorl_b200.cli.train", _cfg(tmp, name, model, dp, foundation, **train), *extra_cli, env=env,
                    timeout=900)
    return _losses(tmp, name), _grads(tmp, name)


def _check(ref, got):
    (rl, rg), (gl, gg) = ref, got
    assert len(rl) == len(gl) == STEPS
    assert rl[0] - min(rl) > 1.0, rl                         # the reference run really learns
    for i, (a, b) in enumerate(zip(rl, gl)):
        # 1 % while the curves are comparable; once the loss has fallen by more than half, bf16 rounding
        # differences between the layouts are amplified by the steep descent (measured: 4 digits agree for
        # six steps, 1.5 % apart at step 11 of a correct run), so later steps get 5 %
        tol = 0.01 * abs(a) if i < 8 else 0.05 * max(abs(a), 2.5)
        assert abs(a - b) < tol, (i, rl, gl)
    assert set(rg) == set(gg) and len(rg) > 10, (sorted(set(rg) ^ set(gg))[:8])
    worst = ("", 0.0)
    for n, g in rg.items():
        rel = float((gg[n].float() - g.float()).norm() / (g.float().norm() + 1e-12))
        if rel > worst[1]:
            worst = (n, rel)
    assert worst[1] < 0.06, worst


CASES = [
    ("fsdp2", 2, 2, dict()),
    ("fsdp2_no_recompute", 2, 2, dict(gradient_checkpointing_method="no_recompute")),
    ("ddp2", 2, 2, dict(data_parallel_mode="ddp")),
    ("hsdp2x2", 4, 4, dict(data_parallel_replicate_size=2, data_parallel_shard_size=2)),
    ("tp2", 2, 1, dict(tensor_parallel_size=2)),
    ("tp2_sp_fused", 2, 1, dict(tensor_parallel_size=2, tensor_parallel_sequence_parallel=True)),
    ("pp2_1f1b", 2, 1, dict(pipeline_parallel_size=2, pipeline_parallel_schedule="1F1B")),
    ("pp2_zbv", 2, 1, dict(pipeline_parallel_size=2, pipeline_parallel_schedule="zbvzerobubble")),
    ("ulysses2", 2, 1, dict(ulysses_parallel_size=2)),
    ("ring2", 2, 1, dict(ringattn_parallel_size=2)),
    ("hybrid2x2", 4, 1, dict(ulysses_parallel_size=2, ringattn_parallel_size=2)),
    ("tp2pp2", 4, 1, dict(tensor_parallel_size=2, pipeline_parallel_size=2,
                          pipeline_parallel_schedule="interleaved1f1b", pipeline_parallel_virtual_stages=2)),
    ("tp4_sp_fused", 4, 1, dict(tensor_parallel_size=4, tensor_parallel_sequence_parallel=True)),
    # data-parallel body, lm-head split by vocabulary rows over the two ranks, tokens pooled for the loss
    ("lm_head_tp2", 2, 2, dict(lm_head_tensor_parallel_size=2)),
]
# model overrides of a case (and of the single-GPU run it is compared with): four-way tensor parallelism
# needs at least four key/value heads
FOUNDATION = {"tp4_sp_fused": {"num_attention_heads": 8, "num_key_value_heads": 4},
              "lm_head_tp2": {"tie_word_embeddings": False}}
_REF = {}


def _reference(tmp_path_factory, model, foundation=None):
    key = (model, tuple(sorted((foundation or {}).items())))
    if key not in _REF:
        _REF[key] = _run(tmp_path_factory.mktemp("ref_" + model.replace("-", "_")), "ref", 1, model=model,
                         foundation=foundation)
    return _REF[key]


@pytest.mark.parametrize("name,nproc,dp,train", CASES, ids=[c[0] for c in CASES])
def test_dense_parallel_modes(tmp_path, tmp_path_factory, name, nproc, dp, train):
    if torch.cuda.device_count() < nproc:
        pytest.skip(f"needs {nproc} GPUs")
    ref = _reference(tmp_path_factory, "small-qwen3", FOUNDATION.get(name))
    got = _run(tmp_path, name, nproc, dp=dp, foundation=FOUNDATION.get(name), **train)
    _check(ref, got)
    if train.get("ringattn_parallel_size", 1) > 1 or train.get("ulysses_parallel_size", 1) > 1:
        # the context-parallel exchanges went through peer memory, not through a collective library
        with open(tmp_path / name / "training_metrics.json") as f:
            calls = json.load(f)["cp_peer_paths"]
        if train.get("ringattn_parallel_size", 1) > 1:
            assert calls["ring_kv_published"] > 0, calls
        if train.get("ulysses_parallel_size", 1) > 1:
            assert calls["ulysses_exchanges"] > 0, calls
    if train.get("tensor_parallel_sequence_parallel"):
        # every collective GEMM of the run went through the single-kernel path
        with open(tmp_path / name / "training_metrics.json") as f:
            calls = json.load(f)["tp_collective_gemms"]
        assert calls["fused"] > 0 and calls["unfused"] == 0, calls   # token counts are multiples of 128


@pytest.mark.parametrize("dispatch", ["alltoall", "fused"])
def test_moe_expert_parallel(tmp_path, tmp_path_factory, dispatch):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    ref = _reference(tmp_path_factory, "small-qwen3-moe")
    got = _run(tmp_path, "ep2", 2, model="small-qwen3-moe", dp=2, extra_cli=("--model.ep_dispatch", dispatch),
               expert_parallel_size=2)
    _check(ref, got)


def test_moe_expert_parallel_block_fp8(tmp_path, tmp_path_factory):
    """Block-scaled fp8 experts under EP 2 against the single-GPU fp8 run (same quantisation on both
    sides), and both within fp8 distance of the bf16 run."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    fp8 = dict(enable_fp8_training=True, fp8_training_allow_blackwell=True, fp8_training_target_modules=["experts"])
    ref = _run(tmp_path, "ref_fp8", 1, model="small-qwen3-moe", **fp8)
    got = _run(tmp_path, "ep2_fp8", 2, model="small-qwen3-moe", dp=2, extra_cli=("--model.ep_dispatch", "fused"),
               expert_parallel_size=2, **fp8)
    _check(ref, got)
    bf16 = _reference(tmp_path_factory, "small-qwen3-moe")[0]
    assert abs(ref[0][0] - bf16[0]) < 0.02 * bf16[0] and abs(ref[0][-1] - bf16[-1]) < 0.15 * bf16[-1] + 0.3


def test_moe_expert_parallel_lora(tmp_path):
    """Adapters over a MoE model whose frozen experts are split over two GPUs (hybrid-shared expert adapters:
    per-expert factors live with their experts, shared factors are replicated): the loss curve and the
    adapter gradients of the one-GPU run."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    lora = ("--lora.enable_lora", "true", "--lora.lora_rank", "8", "--lora.lora_alpha", "16",
            "--lora.moe_hybrid_shared_lora", "true", "--lora.lora_b_init_std", "0.02")
    (rl, rg) = _run(tmp_path, "ref_lora", 1, model="small-qwen3-moe", extra_cli=lora, lr=5e-3)
    (gl, gg) = _run(tmp_path, "ep2_lora", 2, model="small-qwen3-moe", dp=2, expert_parallel_size=2, lr=5e-3,
                    extra_cli=lora + ("--model.ep_dispatch", "fused"))
    assert len(rl) == len(gl) == STEPS and rl[0] - min(rl) > 0.1, rl
    for i, (a, b) in enumerate(zip(rl, gl)):
        assert abs(a - b) < (0.01 if i < 8 else 0.05) * abs(a), (i, rl, gl)
    assert set(rg) == set(gg) and rg and all("lora" in n for n in rg), sorted(set(rg) ^ set(gg))[:8]
    worst = max(((n, float((gg[n].float() - g.float()).norm() / (g.float().norm() + 1e-12))) for n, g in rg.items()),
                key=lambda t: t[1])
    assert worst[1] < 0.06, worst


def test_checkpoint_resume_on_gpu(tmp_path):
    """Pieces of the flat shards written from device memory, read back into them: a run resumed from
    step 2 repeats steps 3 and 4 of the uninterrupted run (the kernels are deterministic)."""
    from dist_utils import run_distributed
    n = min(2, torch.cuda.device_count())
    common = dict(max_steps=4)
    run_distributed("-m", n, "xorl_b200.cli.train", _cfg(tmp_path, "full", dp=n, save_steps=2, **common), env=ENV,
                    timeout=600)
    full = _losses(tmp_path, "full")
    ckpt = tmp_path / "full" / "checkpoints" / "global_step_2"
    assert (ckpt / ".metadata").exists()
    run_distributed("-m", n, "xorl_b200.cli.train",
                    _cfg(tmp_path, "resumed", dp=n, load_checkpoint_path=str(ckpt), **common), env=ENV, timeout=600)
    got = _losses(tmp_path, "resumed")
    assert len(got) >= 2
    for a, b in zip(full[2:], got[-2:]):
        assert abs(a - b) <= 2e-3 * abs(a), (full, got)


def test_checkpoint_written_on_two_gpus_resumes_on_one(tmp_path):
    """ZeRO over two GPUs writes its pieces (plans gathered over NCCL); one GPU, which holds every
    parameter whole, reads them back and continues the same loss curve (same global batch per step)."""
    from dist_utils import run_distributed
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    run_distributed("-m", 2, "xorl_b200.cli.train", _cfg(tmp_path, "two", dp=2, max_steps=4, save_steps=2), env=ENV,
                    timeout=600)
    full = _losses(tmp_path, "two")
    ckpt = tmp_path / "two" / "checkpoints" / "global_step_2"
    assert (ckpt / ".metadata").exists()
    run_distributed("-m", 1, "xorl_b200.cli.train",
                    _cfg(tmp_path, "one", dp=1, max_steps=4, load_checkpoint_path=str(ckpt)), env=ENV, timeout=600)
    got = _losses(tmp_path, "one")
    assert len(got) >= 2
    for a, b in zip(full[2:], got[-2:]):
        assert abs(a - b) <= 0.01 * abs(a), (full, got)
