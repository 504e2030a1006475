"""The trainer end to end on one GPU through the CLI entry point: feature combinations whose device paths
differ from the host ones (activation offload through pinned memory, Hugging Face export and import with the
multi-stream reader, fp8 linears, LoRA with PEFT export, z-loss + router loss on a MoE model, kept
activations).  Each run must learn, write its artifacts and leave the kernels' status words clean."""
import json
import os
import subprocess
import sys

import pytest
import torch
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
pytestmark = pytest.mark.gpu
STEPS = 14


def _run(tmp, name, model="small-qwen3", model_extra=None, lora=None, **train):
    cfg = {
        "model": {"config_path": model, **(model_extra or {})},
        # 16 samples -> four rows of 2048 tokens, all four in every optimizer step: the runs memorise them
        "data": {"datasets": [{"path": "random", "type": "tokenized", "max_seq_len": 700, "min_seq_len": 400,
                               "num_samples": 16}],
                 "sample_packing_sequence_len": 2048, "pad_to_multiple_of": 128, "shuffle_merged_datasets": False},
        "train": {"output_dir": str(tmp / name), "lr": 1e-3, "max_steps": STEPS, "use_wandb": False,
                  "save_hf_weights": False, "save_epochs": 0, "num_train_epochs": 1000, "weight_decay": 0.0,
                  "gradient_accumulation_steps": 4, **train},
    }
    if lora:
        cfg["lora"] = lora
    p = tmp / f"{name}.yaml"
    p.write_text(yaml.safe_dump(cfg))
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "xorl_b200.cli.train", str(p)], env=env, capture_output=True,
                       text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    with open(tmp / name / "training_metrics.json") as f:
        return json.load(f)


def test_activation_offload_matches_the_plain_run(tmp_path):
    plain = _run(tmp_path, "plain")["loss_history"]
    off = _run(tmp_path, "offload", enable_activation_offload=True)["loss_history"]
    assert min(plain) < plain[0] - 0.3, plain
    assert plain == off, (plain, off)                    # moving saved inputs through host memory changes no bit


def test_kept_activations_and_hf_round_trip(tmp_path):
    m = _run(tmp_path, "keep", gradient_checkpointing_method="no_recompute", save_hf_weights=True, save_steps=STEPS)
    assert min(m["loss_history"]) < m["loss_history"][0] - 0.3, m["loss_history"]
    hf = tmp_path / "keep" / f"global_step_{STEPS}" / "hf_ckpt"
    assert any(f.endswith(".safetensors") for f in os.listdir(hf))
    # a second run that starts from the exported weights (multi-stream reader) begins trained, not at ln(V)
    first = _run(tmp_path, "reload", model_extra={"model_path": str(hf)}, max_steps=1, lr=1e-9,
                 load_weights_mode="all_ranks")["loss_history"][0]
    assert first < m["loss_history"][0] - 0.3, (first, m["loss_history"])


def test_fp8_linears_lora_and_moe_losses(tmp_path):
    f8 = _run(tmp_path, "fp8", enable_fp8_training=True, fp8_training_allow_blackwell=True)["loss_history"]
    bf = _run(tmp_path, "bf16")["loss_history"]
    assert min(f8) < f8[0] - 0.3 and abs(f8[-1] - bf[-1]) < 0.1 * abs(bf[-1]), (f8, bf)
    lo = _run(tmp_path, "lora", lora={"enable_lora": True, "lora_rank": 8, "lora_alpha": 16}, lr=5e-3,
              save_hf_weights=True, save_steps=STEPS)
    assert lo["loss_history"][-1] < lo["loss_history"][0]
    peft = tmp_path / "lora" / f"global_step_{STEPS}" / "hf_ckpt"
    assert os.path.exists(peft / "adapter_config.json") and any("adapter_model" in f for f in os.listdir(peft))
    moe = _run(tmp_path, "moe", model="small-qwen3-moe", softmax_auxiliary_loss=True, auxiliary_loss_multiplier=1e-4)
    assert moe["loss_history"][-1] < moe["loss_history"][0]


def test_test_dataset_is_evaluated_at_checkpoints(tmp_path):
    """``data.test_datasets`` = the training rows themselves: the evaluation pass (no gradients, parameters
    gathered unit by unit, fused lm-head log-probabilities) sees the loss the run has memorised them to."""
    p = tmp_path / "ev"
    cfg_extra = {"test_datasets": [{"path": "random", "type": "tokenized", "max_seq_len": 700, "min_seq_len": 400,
                                    "num_samples": 16}]}
    cfg = {
        "model": {"config_path": "small-qwen3"},
        "data": {"datasets": [{"path": "random", "type": "tokenized", "max_seq_len": 700, "min_seq_len": 400,
                               "num_samples": 16}],
                 "sample_packing_sequence_len": 2048, "pad_to_multiple_of": 128, "shuffle_merged_datasets": False,
                 **cfg_extra},
        "train": {"output_dir": str(p), "lr": 1e-3, "max_steps": STEPS, "use_wandb": False, "save_hf_weights": False,
                  "save_epochs": 0, "num_train_epochs": 1000, "weight_decay": 0.0, "gradient_accumulation_steps": 4,
                  "save_steps": 7},
    }
    (tmp_path / "ev.yaml").write_text(yaml.safe_dump(cfg))
    env = dict(os.environ, PYTHONPATH=ROOT + os.pathsep + os.environ.get("PYTHONPATH", ""))
    r = subprocess.run([sys.executable, "-m", "xorl_b200.cli.train", str(tmp_path / "ev.yaml")], env=env,
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    with open(p / "training_metrics.json") as f:
        m = json.load(f)
    ev = m["eval_history"]
    assert [e["step"] for e in ev] == [7, 14] and ev[1]["eval_loss"] < ev[0]["eval_loss"]
    # the evaluation set also holds the rows that the training steps drop (a step takes four packed rows, the
    # ragged rest of an epoch is dropped), so its loss stays above the training loss but well below the start
    assert ev[0]["eval_tokens"] == ev[1]["eval_tokens"] > 4 * 1024
    assert m["loss_history"][-1] - 0.1 < ev[1]["eval_loss"] < m["loss_history"][0] - 0.5, (ev, m["loss_history"])
