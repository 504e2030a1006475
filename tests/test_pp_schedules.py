"""All six pipeline schedules: every (micro-batch, stage) runs F, backward and weight work exactly
once, the order is dead-lock free, and bubbles shrink as expected."""
import pytest

from xorl_b200.parallel.pp_schedules import (SCHEDULES, analytic_bubble_fraction, build_schedule,
                                             estimate_p2p_bytes_per_step, num_chunks, simulate,
                                             stage_owner, global_stage)


@pytest.mark.parametrize("schedule", SCHEDULES)
@pytest.mark.parametrize("pp,n_mb", [(2, 4), (2, 16), (4, 8), (4, 16), (8, 16)])
def test_schedule_is_valid(schedule, pp, n_mb):
    acts = build_schedule(schedule, pp, n_mb, 2)
    res = simulate(acts, schedule, pp, n_mb, 2)
    assert 0.0 <= res["bubble_fraction"] < 0.6


def test_zero_bubble_beats_1f1b():
    pp, n = 4, 16
    b = {s: simulate(build_schedule(s, pp, n, 2), s, pp, n, 2)["bubble_fraction"] for s in SCHEDULES}
    assert b["interleaved1f1b"] < b["1f1b"]
    assert b["interleavedzerobubble"] < b["interleaved1f1b"]
    assert b["zbvzerobubble"] < b["1f1b"] and b["dualpipev"] < b["1f1b"]
    assert abs(b["1f1b"] - analytic_bubble_fraction("1f1b", pp, n)) < 1e-6


def test_stage_maps_roundtrip():
    for s in SCHEDULES:
        c = num_chunks(s, 2)
        for g in range(4 * c):
            r, k = stage_owner(g, 4, s)
            assert global_stage(r, k, 4, s) == g
    assert estimate_p2p_bytes_per_step(2, 16, 8192, 5120, 2) == 2 * 3 * 16 * 8192 * 5120 * 2 * 2


def test_pp_contract_checks():
    import pytest
    import torch
    from xorl_b200.parallel.pp import assign_layers
    from xorl_b200.parallel.pp_contract import (PPContractError, assert_wire_dtype, validate_layer_identity,
                                                validate_microbatch_metadata, validate_stage_plan)
    validate_stage_plan(assign_layers(13, 2, "interleaved1f1b", 2), 13)
    with pytest.raises(PPContractError, match="cover layers"):
        validate_stage_plan([[0, 1], [3]], 4)
    with pytest.raises(PPContractError, match="cover layers"):
        validate_stage_plan([[2, 3], [0, 1]], 4)

    class L:
        def __init__(self, i):
            self.layer_idx = i
    validate_layer_identity([(4, L(4)), (5, L(5))], [4, 5])
    with pytest.raises(PPContractError, match="layer_idx=0"):
        validate_layer_identity([(4, L(0))], [4])
    assert_wire_dtype(torch.zeros(2, dtype=torch.bfloat16), torch.bfloat16, "x")
    with pytest.raises(PPContractError, match="expected torch.bfloat16"):
        assert_wire_dtype(torch.zeros(2), torch.bfloat16, "activation")
    ok = {"position_ids": torch.arange(8), "cu_seqlens": torch.tensor([0, 3, 8])}
    validate_microbatch_metadata(ok, 0)
    with pytest.raises(PPContractError, match="one document"):
        validate_microbatch_metadata({"position_ids": torch.arange(8), "cu_seqlens": None}, 1)
    with pytest.raises(PPContractError, match="do not delimit"):
        validate_microbatch_metadata({"position_ids": torch.arange(8), "cu_seqlens": torch.tensor([0, 9])}, 2)
