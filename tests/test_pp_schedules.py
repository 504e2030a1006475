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
