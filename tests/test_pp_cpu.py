"""Pipeline parallelism over gloo: every schedule reproduces the single-process loss curve."""
import json
import os
import sys

import pytest
import yaml

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def _cfg(tmp, name, **train):
    cfg = {
        "model": {"config_path": "tiny-qwen3",
                  "foundation": {"num_hidden_layers": 4, "tie_word_embeddings": False}},
        "data": {"datasets": [{"path": "random", "type": "tokenized", "max_seq_len": 120,
                               "min_seq_len": 40, "num_samples": 256}],
                 "sample_packing_sequence_len": 256, "pad_to_multiple_of": 64,
                 "shuffle_merged_datasets": False},
        "train": {"output_dir": str(tmp / name), "lr": 1e-3, "max_steps": 3, "use_wandb": False,
                  "device": "cpu", "save_hf_weights": False, "save_epochs": 0, "gradient_accumulation_steps": 4,
                  "enable_mixed_precision": False, **train},
    }
    p = tmp / f"{name}.yaml"
    p.write_text(yaml.safe_dump(cfg))
    return str(p)


def _losses(tmp, name):
    with open(tmp / name / "training_metrics.json") as f:
        return json.load(f)["loss_history"]


@pytest.mark.distributed
@pytest.mark.parametrize("schedule", ["1F1B", "gpipe", "interleaved1f1b", "interleavedzerobubble",
                                      "zbvzerobubble", "dualpipev"])
def test_pp2_matches_single_process(tmp_path, schedule):
    from dist_utils import run_distributed
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    main([_cfg(tmp_path, "ref")])
    ref = _losses(tmp_path, "ref")
    cfg = _cfg(tmp_path, "pp", pipeline_parallel_size=2, pipeline_parallel_schedule=schedule,
               pipeline_parallel_virtual_stages=2)
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "pp")
    assert len(got) == 3
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (schedule, ref, got)


@pytest.mark.distributed
def test_pp_bubble_profile_is_reported(tmp_path):
    """XORL_PP_BUBBLE_PROFILE=1: measured wait share, the unit-cost estimate and the bytes sent."""
    import json
    from dist_utils import run_distributed
    cfg = _cfg(tmp_path, "prof", pipeline_parallel_size=2, pipeline_parallel_schedule="1f1b",
               data_parallel_mode="none", max_steps=2)
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg, env={"XORL_PP_BUBBLE_PROFILE": "1"})
    with open(tmp_path / "prof" / "training_metrics.json") as f:
        b = json.load(f)["pp_bubble"]
    assert 0.0 <= b["measured_bubble_fraction"] < 1.0 and b["waits"] > 0
    assert abs(b["analytic_bubble_fraction"] - 0.2) < 1e-6          # (P - 1) / (M + P - 1) with P = 2, M = 4
    assert b["p2p_sent_bytes"] > 0
