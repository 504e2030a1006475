"""Tensor parallelism over gloo: TP=2 reproduces the single-process loss curve."""
import json
import os
import sys

import pytest
import yaml

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_pp_cpu import _cfg, _losses  # noqa: E402


@pytest.mark.distributed
def test_tp2_matches_single_process(tmp_path):
    from dist_utils import run_distributed
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    main([_cfg(tmp_path, "ref", max_grad_norm=0.5)])
    ref = _losses(tmp_path, "ref")
    cfg = _cfg(tmp_path, "tp", tensor_parallel_size=2, max_grad_norm=0.5)
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "tp")
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (ref, got)


@pytest.mark.distributed
def test_tp2_sequence_parallel_matches_single_process(tmp_path):
    """Token-sharded residual stream, column linears as all-gather -> GEMM, row linears as
    GEMM -> reduce-scatter (the torch.distributed form of the fused kernels on gloo)."""
    from dist_utils import run_distributed
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    main([_cfg(tmp_path, "ref", max_grad_norm=0.5)])
    ref = _losses(tmp_path, "ref")
    cfg = _cfg(tmp_path, "tpsp", tensor_parallel_size=2, tensor_parallel_sequence_parallel=True,
               max_grad_norm=0.5)
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "tpsp")
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (ref, got)


@pytest.mark.distributed
def test_tp2_pp2_interleaved(tmp_path):
    from dist_utils import run_distributed
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    main([_cfg(tmp_path, "ref")])
    ref = _losses(tmp_path, "ref")
    cfg = _cfg(tmp_path, "tppp", tensor_parallel_size=2, pipeline_parallel_size=2,
               pipeline_parallel_schedule="interleaved1f1b", pipeline_parallel_virtual_stages=2)
    run_distributed("-m", 4, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "tppp")
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (ref, got)


@pytest.mark.distributed
def test_lm_head_only_tp2_matches_plain_data_parallel(tmp_path):
    """``lm_head_tensor_parallel_size=2`` with ``tensor_parallel_size=1``: the body is data parallel, the
    two ranks hold half of the vocabulary rows each and pool their tokens for the loss.  Same loss
    curve as plain data parallelism on the same two ranks, and the checkpoint it writes (the lm-head
    under its full shape) resumes without lm-head parallelism."""
    from dist_utils import run_distributed
    run_distributed("-m", 2, "xorl_b200.cli.train", _cfg(tmp_path, "dp", max_grad_norm=0.5, max_steps=4))
    ref = _losses(tmp_path, "dp")
    cfg = _cfg(tmp_path, "lmtp", lm_head_tensor_parallel_size=2, max_grad_norm=0.5, max_steps=4, save_steps=2,
               save_hf_weights=True)
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "lmtp")
    assert len(got) == 4
    # the Hugging Face export holds the whole lm-head, gathered over the lm-head group
    from safetensors import safe_open
    hf = tmp_path / "lmtp" / "global_step_4" / "hf_ckpt"
    shapes = {}
    for f in os.listdir(hf):
        if f.endswith(".safetensors"):
            with safe_open(str(hf / f), "pt") as fh:
                shapes.update({k: tuple(fh.get_slice(k).get_shape()) for k in fh.keys()})
    assert shapes["lm_head.weight"] == (1024, shapes["model.embed_tokens.weight"][1]), shapes.get("lm_head.weight")
    with open(tmp_path / "lmtp" / "startup_metrics.json") as f:
        assert json.load(f)["lm_head_rows_per_rank"] == 512          # half of the tiny model's 1024 rows
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (ref, got)
    resumed = _cfg(tmp_path, "resumed", max_grad_norm=0.5, max_steps=4,
                   load_checkpoint_path=str(tmp_path / "lmtp" / "checkpoints" / "global_step_2"))
    run_distributed("-m", 2, "xorl_b200.cli.train", resumed)
    for a, b in zip(ref[2:], _losses(tmp_path, "resumed")):
        assert abs(a - b) < 2e-4, (ref, _losses(tmp_path, "resumed"))


@pytest.mark.distributed
def test_fsdp_sharded_lm_head_loss_matches_plain_data_parallel(tmp_path):
    """``fsdp_sharded_lm_head_loss``: the lm-head is never gathered, the loss streams the data-parallel
    group's tokens through each rank's vocabulary rows in ``..._num_chunks`` chunks."""
    from dist_utils import run_distributed
    run_distributed("-m", 2, "xorl_b200.cli.train", _cfg(tmp_path, "dp", max_grad_norm=0.5))
    ref = _losses(tmp_path, "dp")
    cfg = _cfg(tmp_path, "sharded", fsdp_sharded_lm_head_loss=True, fsdp_sharded_lm_head_loss_num_chunks=3,
               max_grad_norm=0.5)
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "sharded")
    with open(tmp_path / "sharded" / "startup_metrics.json") as f:
        assert json.load(f)["lm_head_rows_per_rank"] == 512
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (ref, got)


@pytest.mark.distributed
def test_lm_head_tp2_on_four_ranks_shards_the_head_rows_over_their_replicas(tmp_path):
    """Four data-parallel ranks in two lm-head groups of two: each half of the vocabulary rows lives on two
    ranks (one per group) and is ZeRO-sharded over that pair; gradients of a row reach it from both groups.
    Same loss curve as plain data parallelism over the four ranks."""
    from dist_utils import run_distributed
    run_distributed("-m", 4, "xorl_b200.cli.train", _cfg(tmp_path, "dp4", max_grad_norm=0.5, gradient_accumulation_steps=2))
    ref = _losses(tmp_path, "dp4")
    cfg = _cfg(tmp_path, "lmtp4", lm_head_tensor_parallel_size=2, max_grad_norm=0.5, gradient_accumulation_steps=2)
    run_distributed("-m", 4, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "lmtp4")
    assert len(got) == len(ref) == 3
    for a, b in zip(ref, got):
        assert abs(a - b) < 2e-4, (ref, got)
