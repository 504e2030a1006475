"""Analytical planner: sanity of the estimates against this framework's measured numbers."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def test_single_gpu_estimate_is_near_measured():
    from xorl_b200.models.config import preset
    from xorl_b200.sim import ParallelLayout, estimate
    cfg = preset("qwen3-8b")
    e = estimate(cfg, ParallelLayout(), 4096, doc_lens=[2048, 2048])
    # measured on one B200: 337 ms per 4096-token step, 140 GB peak
    assert 250 < e.step_ms < 450, e.breakdown_ms
    assert 110 < e.memory_gb < 175 and e.fits, e.memory_breakdown_gb
    assert e.breakdown_ms["gemm"] > e.breakdown_ms["attention"] > 0


def test_planner_ranks_feasible_layouts_and_rejects_oversized():
    from xorl_b200.models.config import preset
    from xorl_b200.sim import ParallelLayout, estimate, plan
    cfg8, cfg32 = preset("qwen3-8b"), preset("qwen3-32b")
    best = plan(cfg8, 8, 4096)
    assert best and all(b.fits for b in best) and best[0].layout.world == 8
    assert best[0].tokens_per_s >= best[-1].tokens_per_s
    assert not estimate(cfg32, ParallelLayout(), 8192).fits            # 32B does not fit one GPU
    assert any(e.fits for e in plan(cfg32, 8, 8192))
    moe = preset("qwen3-30b-a3b")
    assert any(e.layout.ep > 1 for e in plan(moe, 8, 4096, top=20))


def test_cli(capsys):
    from xorl_b200.sim.__main__ import main
    out = main(["--model", "qwen3-8b", "--gpus", "8", "--top", "2"])
    assert len(out) == 2 and "fsdp" in out[0]["layout"]
