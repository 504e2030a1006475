"""Trainer diagnostics on CPU: the rank watchdog (a silent peer and a peer that reports a failure,
both made on the host), the non-finite gradient scan, the metrics file."""
import json
import os
import sys
import time

import pytest
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from xorl_b200.utils.diagnostics import (MemoryHistory, MetricsSink, RankFailure, RankWatchdog,  # noqa: E402
                                         nonfinite_gradient_report, nvtx_range)


def test_watchdog_notices_a_rank_that_stops_beating():
    store = dist.HashStore()
    a = RankWatchdog(store, 0, 2, interval_s=0.05, timeout_s=0.4).start()
    b = RankWatchdog(store, 1, 2, interval_s=0.05, timeout_s=0.4).start()
    time.sleep(0.3)
    a.check()
    b.check()
    b.stop()                                   # rank 1 goes silent (its process "hangs")
    deadline = time.time() + 5
    with pytest.raises(RankFailure, match="rank 1 sent no heartbeat"):
        while time.time() < deadline:
            a.check()
            time.sleep(0.05)
    a.stop()


def test_watchdog_relays_a_reported_failure_before_the_timeout():
    store = dist.HashStore()
    a = RankWatchdog(store, 0, 2, interval_s=0.05, timeout_s=60).start()
    b = RankWatchdog(store, 1, 2, interval_s=0.05, timeout_s=60).start()
    b.report_failure("RuntimeError: injected on the host")
    deadline = time.time() + 5
    with pytest.raises(RankFailure, match="rank 1 reported: RuntimeError: injected"):
        while time.time() < deadline:
            a.check()
            time.sleep(0.05)
    a.stop()
    b.stop()


def test_nonfinite_scan_names_the_parameter():
    from xorl_b200.models.config import preset
    from xorl_b200.models.decoder import DecoderLM
    from xorl_b200.parallel.state import get_parallel_state, reset_parallel_state
    from xorl_b200.parallel.zero import Zero3Engine
    reset_parallel_state()
    cfg = preset("tiny-qwen3")
    model = DecoderLM(cfg, dtype=torch.float32, device="meta")
    eng = Zero3Engine(model, get_parallel_state(), compute_dtype=torch.float32, device=torch.device("cpu"), seed=0)
    ids = torch.randint(0, cfg.vocab_size, (64,))
    eng.forward_backward(ids, ids.clone(), cu_seqlens=torch.tensor([0, 64], dtype=torch.int32), grad_scale=1 / 64)
    eng.finish_grad_sync()
    assert nonfinite_gradient_report(eng) == []
    g = eng.units[1].groups[0]
    i, a, b = g.param_segments_in_shard()[2]
    g.grad_shard[a] = float("nan")
    rep = nonfinite_gradient_report(eng)
    assert len(rep) == 1 and rep[0].endswith(g.named_params[i][0]), rep
    reset_parallel_state()


def test_metrics_sink_writes_json_lines_and_helpers_are_inert_on_cpu(tmp_path):
    class T:
        use_wandb, wandb_log_interval, output_dir = False, 2, str(tmp_path)
        wandb_project = wandb_name = wandb_tags = None
    sink = MetricsSink(T, rank=0)
    for step in range(1, 5):
        sink.log({"loss": 1.0 / step, "note": "skipped"}, step)
    sink.close()
    rows = [json.loads(l) for l in open(tmp_path / "metrics.jsonl")]
    assert [r["step"] for r in rows] == [2, 4] and "note" not in rows[0]
    assert MetricsSink(T, rank=1).file is None
    with nvtx_range("x"):
        pass
    mh = MemoryHistory(0, env={"XORL_MEMHIST": "1"})
    assert mh.enabled == torch.cuda.is_available()
    if not mh.enabled:
        assert mh.after_step(2) is None and mh.on_oom() is None
    mh.close()


def test_kernel_pin_is_written_once_and_detects_a_change(tmp_path):
    from xorl_b200.models.numerics import KernelPinError, pin_kernel_configs
    first = pin_kernel_configs(str(tmp_path))
    assert first["mismatch"] == {} and (tmp_path / "kernel_pin.json").exists()
    assert pin_kernel_configs(str(tmp_path), strict=True)["mismatch"] == {}
    pin = json.loads((tmp_path / "kernel_pin.json").read_text())
    pin["native_library_sha256"] = "0" * 64
    (tmp_path / "kernel_pin.json").write_text(json.dumps(pin))
    assert "native_library_sha256" in pin_kernel_configs(str(tmp_path))["mismatch"]
    with pytest.raises(KernelPinError):
        pin_kernel_configs(str(tmp_path), strict=True)


def test_canaries_catch_a_write_past_a_guarded_buffer():
    import torch
    from xorl_b200.utils import canary
    buf = canary.guarded_empty((10, 7), torch.bfloat16, "cpu", "scratch.test", force=True)
    assert buf.shape == (10, 7) and buf.dtype == torch.bfloat16 and buf.data_ptr() % 64 == 0
    buf.fill_(1.0)                                            # writing the whole body is fine
    assert canary.check_all() >= 1
    raw = buf._xb_canary_raw
    raw[canary.GUARD_BYTES + buf.numel() * 2 + 3] = 0         # one byte past the end
    with pytest.raises(RuntimeError, match=r"scratch.test \(past its end\)"):
        canary.check_all()
    raw[canary.GUARD_BYTES + buf.numel() * 2 + 3] = canary.PATTERN
    raw[5] = 1                                                # and one before the start
    with pytest.raises(RuntimeError, match=r"scratch.test \(before its start\)"):
        canary.check_all()
    raw[5] = canary.PATTERN
    del buf, raw
    import gc
    gc.collect()
    canary.check_all()                                        # freed buffers leave the registry
    assert not any(n == "scratch.test" for n, _, _ in canary._registry)
    # off by default: a plain allocation
    plain = canary.guarded_empty((4,), torch.float32, "cpu", "x")
    assert not hasattr(plain, "_xb_canary_raw")
