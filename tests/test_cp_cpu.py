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


def test_peer_exchange_copy_plans_equal_the_all_to_all_layouts():
    """The strided copies of the copy-engine Ulysses exchange, replayed on host byte buffers for every
    rank, give exactly what the all-to-all formulation gives."""
    import numpy as np
    import torch
    from xorl_b200.parallel.sequence_parallel import _PeerExchange
    U, T, h, D, es = 4, 6, 3, 8, 2
    H = U * h
    xs = [torch.randn(T, H, D).to(torch.bfloat16) for _ in range(U)]                    # per-rank inputs

    def replay(pieces_of, srcs, nbytes):
        slots = [np.zeros(nbytes, dtype=np.uint8) for _ in range(U)]
        for r in range(U):
            src = srcs[r].contiguous().view(torch.uint8).reshape(-1).numpy()
            for u, (doff, dpitch, soff, spitch, width, rows) in enumerate(pieces_of(r)):
                for i in range(rows):
                    slots[u][doff + i * dpitch: doff + i * dpitch + width] = src[soff + i * spitch: soff + i * spitch + width]
        return slots

    nbytes = T * H * D * es
    got = replay(lambda r: _PeerExchange.seq_to_head_pieces(r, T, H, D, U, es), xs, nbytes)
    for u in range(U):
        want = torch.cat([xs[r].reshape(T, U, h, D)[:, u] for r in range(U)], 0)          # [U*T, h, D]
        out = torch.from_numpy(got[u]).view(torch.bfloat16).reshape(U * T, h, D)
        assert torch.equal(out, want)
    # and back: [U*T, h, D] on every rank -> [T, U*h, D]
    ys = [torch.randn(U * T, h, D).to(torch.bfloat16) for _ in range(U)]
    got = replay(lambda r: _PeerExchange.head_to_seq_pieces(r, T, h, D, U, es), ys, nbytes)
    for u in range(U):
        want = torch.stack([ys[r].reshape(U, T, h, D)[u] for r in range(U)], 1).reshape(T, U * h, D)
        out = torch.from_numpy(got[u]).view(torch.bfloat16).reshape(T, U * h, D)
        assert torch.equal(out, want)
