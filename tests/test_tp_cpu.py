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
