"""Context parallelism over gloo: Ulysses, zigzag ring and the hybrid reproduce the
single-process loss curve."""
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
from test_pp_cpu import _cfg, _losses  # noqa: E402


@pytest.mark.distributed
@pytest.mark.parametrize("ulysses,ring", [(2, 1), (1, 2), (2, 2)])
def test_cp_matches_single_process(tmp_path, ulysses, ring):
    from dist_utils import run_distributed
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    main([_cfg(tmp_path, "ref", gradient_accumulation_steps=2)])
    ref = _losses(tmp_path, "ref")
    cfg = _cfg(tmp_path, "cp", ulysses_parallel_size=ulysses, ringattn_parallel_size=ring,
               gradient_accumulation_steps=2)
    run_distributed("-m", ulysses * ring, "xorl_b200.cli.train", cfg)
    got = _losses(tmp_path, "cp")
    for a, b in zip(ref, got):
        assert abs(a - b) < 3e-4, (ref, got)


def test_zigzag_indices_cover_document():
    import numpy as np
    from xorl_b200.data import zigzag_indices
    L, cp = 64, 4
    allidx = np.concatenate([zigzag_indices(L, cp, r) for r in range(cp)])
    assert sorted(allidx.tolist()) == list(range(L))
    assert zigzag_indices(L, cp, 0).tolist() == list(range(0, 8)) + list(range(56, 64))


@pytest.mark.distributed
@pytest.mark.parametrize("preset", ["tiny-qwen3-5", "tiny-nemotron-h"])
def test_gated_deltanet_family_under_ulysses(tmp_path, preset):
    """Hybrid families (GatedDeltaNet + gated attention; Mamba2 + rotary-free attention + MoE) with
    every document cut across two sequence-parallel ranks: same losses as one process."""
    import yaml
    from dist_utils import run_distributed
    from xorl_b200.cli.train import main
    from xorl_b200.parallel.state import reset_parallel_state

    def cfg(name, **train):
        path = _cfg(tmp_path, name, **train)
        c = yaml.safe_load(open(path))
        c["model"] = {"config_path": preset, "foundation": {"tie_word_embeddings": False}}
        open(path, "w").write(yaml.safe_dump(c))
        return path
    reset_parallel_state()
    main([cfg("gdn_ref", gradient_accumulation_steps=2)])
    ref = _losses(tmp_path, "gdn_ref")
    run_distributed("-m", 2, "xorl_b200.cli.train", cfg("gdn_cp", ulysses_parallel_size=2, gradient_accumulation_steps=2))
    got = _losses(tmp_path, "gdn_cp")
    for a, b in zip(ref, got):
        assert abs(a - b) < 3e-4, (ref, got)
