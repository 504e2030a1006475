"""Analytical planner: sanity of the estimates against this framework's measured numbers."""
import os
import sys

import pytest

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


def test_calibration_packs_discovery_validation_and_fit(tmp_path):
    import json
    from xorl_b200.sim import calibration_packs as C
    from xorl_b200.sim.__main__ import main
    names = C.list_calibration_packs()
    assert {"b200_qwen3_8b", "b200_qwen3_30b_a3b"} <= set(names)
    pack = C.load_pack("builtin:b200_qwen3_8b")
    ev = C.evaluate_pack(pack)
    assert len(ev["runs"]) == 3 and ev["mean_abs_relative_error"] < 0.08        # the shipped coefficients fit their runs
    # a deliberately wrong coefficient is pulled back by the fit
    bad = C.CalibrationPack("bad", None, dict(pack.manifest, coefficients=dict(pack.coefficients, gemm_eff=0.3)))
    assert C.evaluate_pack(bad)["mean_signed_relative_error"] > 0.5
    fit = C.fit_coefficient(bad, "gemm_eff", 0.2, 1.0)
    assert abs(fit["value"] - pack.coefficients["gemm_eff"]) < 0.05
    assert abs(fit["evaluation"]["mean_signed_relative_error"]) < 1e-3
    # validation: unknown coefficients, missing fields and machine-specific content are refused
    m = json.loads(json.dumps(pack.manifest))
    m["coefficients"]["warp_speed"] = 9.0
    with pytest.raises(ValueError, match="unknown coefficients"):
        C.validate_manifest(m, list(__import__("xorl_b200.sim.planner", fromlist=["x"]).default_b200_pack()))
    m = json.loads(json.dumps(pack.manifest))
    m["observed_runs"][0]["source"] = "kubectl exec trainer -- python bench.py"
    with pytest.raises(ValueError, match="not portable"):
        C.validate_manifest(m)
    m = json.loads(json.dumps(pack.manifest))
    del m["observed_runs"][0]["step_ms"]
    with pytest.raises(ValueError, match="lacks 'step_ms'"):
        C.validate_manifest(m)
    # a bare JSON of overrides still works as --calibration, and the CLI evaluates a built-in pack
    p = tmp_path / "c.json"
    p.write_text(json.dumps({"gemm_eff": 0.5}))
    assert C.load_pack(str(p)).coefficients == {"gemm_eff": 0.5}
    out = main(["--calibration", "builtin:b200_qwen3_30b_a3b", "--evaluate"])
    assert abs(out["runs"][0]["relative_error"]) < 0.05
    assert main(["--model", "qwen3-8b", "--gpus", "8", "--calibration", str(p), "--top", "2"])
