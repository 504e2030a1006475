"""Training service on CPU: REST contract with the dummy backend (ordering, failure injection,
sessions, auth), a real tiny model behind the same routes, weight sync transports, the ZMQ remote
backend and the sparse-delta codec."""
import os
import sys
import threading
import time

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from fastapi.testclient import TestClient  # noqa: E402

from xorl_b200.server.api_server import ServerState, create_app  # noqa: E402
from xorl_b200.server.backend import DummyBackend, LocalBackend  # noqa: E402
from xorl_b200.server.future_store import FutureStore  # noqa: E402
from xorl_b200.server.orchestrator import (Orchestrator, OrchestratorRequest, RequestProcessor,  # noqa: E402
                                           SeqIdAwareFIFOPolicy)
from xorl_b200.server import packing  # noqa: E402


def _datum(n, start=1):
    toks = list(range(start, start + n))
    return {"model_input": {"tokens": toks},
            "loss_fn_inputs": {"target_tokens": {"data": toks[1:] + [-100], "dtype": "int64"}}}


def _poll(client, rid, timeout=30.0):
    t0 = time.time()
    while time.time() - t0 < timeout:
        r = client.post("/api/v1/retrieve_future", json={"request_id": rid}).json()
        if r.get("type") != "try_again":
            return r
        time.sleep(0.01)
    raise AssertionError("future never resolved")


def test_future_store_ttl_and_abort():
    fs = FutureStore(ttl_seconds=10)
    a, b = fs.create("x"), fs.create("y")
    fs.set_result(a, {"ok": 1})
    assert fs.get(a)["state"] == "done" and fs.pending() == 1
    assert fs.abort(b) and not fs.abort(b)
    fs.set_result(b, 1)                       # late result of an aborted request is dropped
    assert fs.get(b)["state"] == "failed"
    assert fs.cleanup(now=time.time() + 100) == 2 and fs.get(a) is None


def test_packing_and_dp_balance():
    lengths = [100, 900, 500, 300, 700, 50]
    for fn in (packing.pack_sequential, packing.pack_best_fit):
        bins = fn(lengths, 1000)
        assert sorted(i for b in bins for i in b) == list(range(6))
        assert all(sum(lengths[i] for i in b) <= 1000 for b in bins)
    assert len(packing.pack_best_fit(lengths, 1000)) <= len(packing.pack_sequential(lengths, 1000))
    plan = packing.balance_across_dp(packing.pack_best_fit(lengths, 1000), lengths, 2)
    assert len(plan) == 2 and len(plan[0]) == len(plan[1])      # equal micro-batch counts per rank
    mb = packing.datums_to_micro_batch([{"tokens": [5, 6, 7], "target_tokens": [6, 7, -100]},
                                        {"tokens": [1, 2], "weights": [1.0, 0.0]}], pad_to=8)
    assert mb["input_ids"].numel() == 8 and mb["cu_seqlens"].tolist() == [0, 3, 5, 8]
    assert mb["num_valid_tokens"] == 3 and mb["position_ids"][:5].tolist() == [0, 1, 2, 0, 1]


def test_balanced_dp_packer_and_oversized_policy():
    from xorl_b200.server.orchestrator import RequestProcessor
    lengths = [900, 850, 400, 380, 300, 250, 120, 100]
    bins = packing.pack_balanced_dp(lengths, 1000, dp=4)
    assert len(bins) % 4 == 0 and all(bins)                       # k*dp bins, none empty: no dummy batches
    assert sorted(i for b in bins for i in b) == list(range(8))
    loads = [sum(lengths[i] for i in b) for b in bins]
    assert max(loads) <= 1000 and max(loads) - min(loads) <= 300
    plan = RequestProcessor(4, 1000, "balanced_dp").plan([{"tokens": [0] * n} for n in lengths])
    assert all(len(r) == 1 and r[0] for r in plan)
    # fewer samples than ranks: best-fit, the dispatcher pads with dummy batches
    assert packing.pack_balanced_dp([10, 20], 100, dp=4) == packing.pack_best_fit([10, 20], 100)
    datums = [{"tokens": [1, 2, 3], "weights": [1.0, 1.0, 0.0]}, {"tokens": list(range(9)), "weights": [1.0] * 9,
                                                                   "tag": "x"}]
    with pytest.raises(ValueError, match="datum 1 has 9 tokens"):
        packing.apply_oversized_policy(datums, 4, "error")
    kept, origin = packing.apply_oversized_policy(datums, 4, "skip")
    assert origin == [0] and kept[0] is datums[0]
    kept, origin = packing.apply_oversized_policy(datums, 4, "truncate")
    assert origin == [0, 1] and kept[1]["tokens"] == [0, 1, 2, 3] and len(kept[1]["weights"]) == 4 and kept[1]["tag"] == "x"
    rp = RequestProcessor(1, 4, "sequential", on_oversized="skip")
    kept, origin = rp.admit(datums)
    res = rp.restore_order({"loss": 1.0, "logprobs": [[0.1, 0.2, 0.3]]}, origin, 2)
    assert res["logprobs"] == [[0.1, 0.2, 0.3], []] and res["skipped_datums"] == [1]
    with pytest.raises(ValueError):
        RequestProcessor(1, 4, "unknown")


def test_seq_id_policy_reorders():
    p = SeqIdAwareFIFOPolicy(max_wait=60)
    for s in (2, 0, 1):
        p.push(OrchestratorRequest(request_id=str(s), op="x", seq_id=s))
    assert [p.pop().seq_id for _ in range(3)] == [0, 1, 2]
    p.push(OrchestratorRequest(request_id="late", op="x", seq_id=5))
    assert p.pop() is None                                     # seq 3, 4 not seen yet
    p.push(OrchestratorRequest(request_id="n", op="x"))
    assert p.pop().request_id == "n"                           # un-numbered requests never wait


def test_orchestrator_failure_injection():
    done = {}
    be = DummyBackend(failure_rate=1.0)
    o = Orchestrator(be, on_result=lambda rid, res, err: done.__setitem__(rid, (res, err)))
    o.start()
    o.submit(OrchestratorRequest(request_id="a", op="optim_step"))
    t0 = time.time()
    while "a" not in done and time.time() - t0 < 5:
        time.sleep(0.01)
    o.stop()
    assert done["a"][0] is None and "injected failure" in done["a"][1]


def test_rest_contract_dummy_backend(tmp_path):
    be = DummyBackend(processing_delay=0.05)
    st = ServerState(be, str(tmp_path), packing_len=64, api_keys=["k1"], session_timeout=0.5)
    with TestClient(create_app(st)) as c:
        assert c.get("/health").json()["status"] == "ok"
        assert c.post("/api/v1/optim_step", json={}).status_code == 401
        c.headers["x-api-key"] = "k1"
        # out-of-order seq ids are executed in order (both queue up behind a busy backend)
        c.post("/api/v1/abort_gradient_epoch", json={})
        c.post("/api/v1/save_weights", json={})
        r2 = c.post("/api/v1/optim_step", json={"seq_id": 1}).json()
        r1 = c.post("/api/v1/forward_backward", json={"seq_id": 0, "forward_backward_input":
                                                      {"data": [_datum(10), _datum(7)]}}).json()
        out1, out2 = _poll(c, r1["request_id"]), _poll(c, r2["request_id"])
        assert be.calls[-2:] == ["forward_backward", "optim_step"]
        assert out1["type"] == "forward_backward" and len(out1["loss_fn_outputs"]) == 2
        assert out1["loss_fn_outputs"][0]["logprobs"]["shape"] == [10]
        assert out2["type"] == "optim_step" and out2["metrics"]["step"] == 1.0
        # a datum longer than the packing length fails as a user error
        bad = c.post("/api/v1/forward_backward", json={"forward_backward_input": {"data": [_datum(100)]}}).json()
        res = _poll(c, bad["request_id"])
        assert res["type"] == "request_failed" and res["category"] == "user"
        assert c.post("/api/v1/forward_backward", json={"forward_backward_input": {"data": []}}).status_code == 422
        assert c.post("/api/v1/retrieve_future", json={"request_id": "nope"}).status_code == 404
        assert c.post("/api/v1/optim_step", json={"model_id": "ghost"}).status_code == 404
        # sessions own models and release them on expiry
        sid = c.post("/api/v1/create_session", json={"tags": ["t"]}).json()["session_id"]
        mid = c.post("/api/v1/create_model", json={"session_id": sid, "lora_config": {"rank": 4}}).json()["model_id"]
        assert c.post("/api/v1/session_heartbeat", json={"session_id": sid}).json()["ok"]
        assert any(r["training_run_id"] == mid for r in c.get("/api/v1/training_runs").json()["training_runs"])
        time.sleep(0.6)
        assert c.get("/api/v1/session_info").json()["sessions"] == []
        assert c.post("/api/v1/optim_step", json={"model_id": mid}).status_code == 404
        # inference endpoints and sleep / wake
        assert c.post("/add_inference_endpoint", json={"url": "http://169.254.169.254:80"}).status_code == 422
        assert c.post("/add_inference_endpoint", json={"url": "ftp://127.0.0.1:21"}).status_code == 422
        assert c.post("/api/v1/create_model", json={"model_id": "../escape"}).status_code == 422
        c.post("/add_inference_endpoint", json={"url": "http://127.0.0.1:30000", "world_size": 2})
        assert c.get("/list_inference_endpoints").json()["endpoints"][0]["world_size"] == 2
        assert c.post("/api/v1/create_sampling_session", json={}).json()["endpoint"] == "http://127.0.0.1:30000"
        assert c.post("/remove_inference_endpoint", json={"url": "http://127.0.0.1:30000"}).status_code == 200
        assert c.post("/api/v1/set_sync_quantization", json={"format": "fp8"}).json()["format"] == "fp8"
        assert c.post("/sleep").json()["asleep"] and c.get("/health").json()["asleep"]
        assert not c.post("/wake_up").json()["asleep"]


def test_rest_failures_surface_as_request_failed(tmp_path):
    st = ServerState(DummyBackend(failure_rate=1.0), str(tmp_path))
    with TestClient(create_app(st)) as c:
        rid = c.post("/api/v1/optim_step", json={}).json()["request_id"]
        out = _poll(c, rid)
        assert out["type"] == "request_failed" and out["category"] == "server"
        assert c.get("/health").json()["pending"] == 0


@pytest.fixture()
def tiny_runner(tmp_path):
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    sa = ServerArguments(model_preset="tiny-qwen3", output_dir=str(tmp_path / "srv"), device="cpu",
                         sample_packing_sequence_len=256, enable_mixed_precision=False)
    runner = ModelRunner(Trainer(sa.to_trainer_arguments()))
    yield runner
    reset_parallel_state()


def test_local_backend_trains_and_restores(tmp_path, tiny_runner):
    st = ServerState(LocalBackend(tiny_runner), tiny_runner.output_dir, packing_len=256)
    data = [_datum(40, 3), _datum(25, 50), _datum(60, 7)]
    with TestClient(create_app(st)) as c:
        def fb(kind="forward_backward", key="forward_backward_input", loss_fn="cross_entropy", d=data, cfg=None):
            rid = c.post(f"/api/v1/{kind}", json={key: {"data": d, "loss_fn": loss_fn,
                                                        "loss_fn_config": cfg or {}}}).json()["request_id"]
            return _poll(c, rid, 120)
        losses = []
        for step in range(4):
            out = fb()
            assert out["type"] == "forward_backward", out
            losses.append(out["metrics"]["loss:sum"])
            o = _poll(c, c.post("/api/v1/optim_step", json={"adam_params": {"learning_rate": 5e-3},
                                                            "gradient_clip": 1.0}).json()["request_id"], 120)
            assert o["metrics"]["step"] == step + 1 and o["metrics"]["grad_norm"] > 0
        assert losses[-1] < losses[0]
        lp0 = out["loss_fn_outputs"][0]["logprobs"]["data"]
        assert len(lp0) == 40 and all(v <= 0 for v in lp0[:-1])
        # forward-only log-probs agree with what the next forward_backward reports
        f = fb("forward", "forward_input")
        saved = _poll(c, c.post("/api/v1/save_weights", json={"path": "ckpt_a"}).json()["request_id"], 120)
        assert saved["path"] == "xorl://default/weights/ckpt_a"
        assert [x["name"] for x in c.get("/api/v1/list_checkpoints").json()["checkpoints"]] == ["ckpt_a"]
        out5 = fb()
        a = f["loss_fn_outputs"][1]["logprobs"]["data"]
        b = out5["loss_fn_outputs"][1]["logprobs"]["data"]
        assert max(abs(x - y) for x, y in zip(a, b)) < 1e-4
        _poll(c, c.post("/api/v1/optim_step", json={"adam_params": {"learning_rate": 5e-3}}).json()["request_id"], 120)
        moved = fb("forward", "forward_input")["loss_fn_outputs"][1]["logprobs"]["data"]
        assert max(abs(x - y) for x, y in zip(a, moved)) > 1e-4
        # restoring the checkpoint restores the log-probs
        r = _poll(c, c.post("/api/v1/load_weights", json={"path": "xorl://default/weights/ckpt_a"}).json()["request_id"], 120)
        assert r["type"] == "load_weights", r
        back = fb("forward", "forward_input")["loss_fn_outputs"][1]["logprobs"]["data"]
        assert max(abs(x - y) for x, y in zip(a, back)) < 1e-5
        # log-probabilities on the sampler's support: top_k = 1 leaves one token, so a label is either
        # certain (0) or outside the support (-inf); wider filters only raise a kept label's value
        top1 = fb("forward", "forward_input", cfg={"top_k": 1})
        v1 = top1["loss_fn_outputs"][1]["logprobs"]["data"][:-1]
        assert all(x == 0.0 or x <= -1e29 for x in v1)
        assert top1["metrics"]["out_of_support_tokens"] == sum(
            x <= -1e29 for o in top1["loss_fn_outputs"] for x in o["logprobs"]["data"])
        wide = fb("forward", "forward_input", cfg={"top_p": 0.999, "temperature": 1.0})
        vw = wide["loss_fn_outputs"][1]["logprobs"]["data"][:-1]
        assert all(w >= x - 1e-5 for w, x in zip(vw, back[:-1]) if w > -1e29)
        # a policy-gradient loss through the same route
        rl = [dict(d) for d in data]
        for d in rl:
            n = len(d["model_input"]["tokens"])
            d["loss_fn_inputs"] = dict(d["loss_fn_inputs"], logprobs={"data": [-2.0] * n, "dtype": "float32"},
                                       advantages={"data": [0.5] * n, "dtype": "float32"})
        o = fb(loss_fn="importance_sampling", d=rl)
        assert o["type"] == "forward_backward", o
        # an optim_step with nothing accumulated is refused; bad token ids are a user error
        _poll(c, c.post("/api/v1/abort_gradient_epoch", json={}).json()["request_id"])
        e = _poll(c, c.post("/api/v1/optim_step", json={}).json()["request_id"])
        assert e["type"] == "request_failed"
        badd = {"model_input": {"tokens": [1, 10 ** 7]}, "loss_fn_inputs": {}}
        e = fb(d=[badd])
        assert e["type"] == "request_failed" and e["category"] == "user"
        assert c.post("/api/v1/delete_checkpoint", json={"name": "ckpt_a"}).json()["deleted"] == "ckpt_a"


def test_weight_sync_transports(tmp_path, tiny_runner):
    from safetensors.torch import load_file
    from xorl_b200.server import weight_sync as ws
    h = ws.WeightSyncHandler(tiny_runner)
    out = h.sync(backend="file", directory=str(tmp_path / "w"), bucket_size_mb=1)
    assert out["synced"] and out["buckets"] >= 1 and os.path.exists(out["index"])
    got = {}
    for f in sorted(os.listdir(tmp_path / "w")):
        if f.endswith(".safetensors"):
            got.update(load_file(str(tmp_path / "w" / f)))
    assert "model.layers.0.self_attn.q_proj.weight" in got and "model.layers.0.mlp.up_proj.weight" in got
    assert not any("qkv_proj" in k or "gate_up_proj" in k for k in got)
    # sparse delta: first generation full, the second only carries what one step changed
    d1 = h.sync(backend="sparse_delta", directory=str(tmp_path / "d"))
    weights = ws.apply_delta_generation(str(tmp_path / "d" / "gen-000001"), {})
    tiny_runner.forward_backward("default", [{"tokens": list(range(1, 30))}], None)
    tiny_runner.optim_step("default", adam_params={"learning_rate": 1e-5})
    d2 = h.sync(backend="sparse_delta", directory=str(tmp_path / "d"))
    assert d2["delta_stats"]["bytes"] < d1["delta_stats"]["bytes"]
    ws.apply_delta_generation(str(tmp_path / "d" / "gen-000002"), weights)
    ref = dict(ws.iter_sync_tensors(tiny_runner.engine, tiny_runner.model.config))
    for k, v in ref.items():
        assert torch.equal(weights[k], v.cpu()), k
    # bucket flattening round trip and the peer-copy transport on host memory
    bucket = [("a", torch.randn(3, 5).bfloat16()), ("b", torch.arange(7, dtype=torch.uint8))]
    flat, man = ws.flatten_bucket(bucket)
    back = ws.unflatten_bucket(flat, man)
    assert torch.equal(back["a"], bucket[0][1]) and torch.equal(back["b"], bucket[1][1])
    dst = torch.zeros(flat.numel(), dtype=torch.uint8)
    ws.PeerCopyTransport(dst.data_ptr(), dst.numel()).send_bucket(bucket)
    assert torch.equal(dst, flat)
    # fp8 sync quantisation emits scale companions for 128-aligned matrices only
    q = ws._quantise("x.q_proj.weight", torch.randn(128, 256), "fp8")
    assert [n for n, _ in q] == ["x.q_proj.weight", "x.q_proj.weight_scale_inv"] and q[0][1].dtype == torch.uint8


@pytest.mark.parametrize("preset_name", ["tiny-qwen3", "tiny-qwen3-moe"])
def test_lora_policy_is_synced_with_its_adapter_folded_in(tmp_path, preset_name):
    """The inference engine gets plain Hugging Face weights: base + scaling * B A (fused projections per
    slice, stacked experts per expert).  A model loaded from the synced files without any adapter gives the
    trained adapter model's log-probabilities; the engine's own base weights are untouched."""
    from safetensors.torch import load_file
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server import weight_sync as ws
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    targets = ["q_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]
    sa = ServerArguments(model_preset=preset_name, output_dir=str(tmp_path / "srv"), device="cpu",
                         sample_packing_sequence_len=256, enable_mixed_precision=False, enable_lora=True,
                         lora_rank=4, lora_alpha=8, lora_target_modules=targets)
    r = ModelRunner(Trainer(sa.to_trainer_arguments()))
    data = [{"tokens": list(range(3, 60))}]
    base_lp = r.forward("default", data, None)["logprobs"][0]
    for _ in range(3):
        r.forward_backward("default", data, None)
        r.optim_step("default", adam_params={"learning_rate": 2e-2})
    tuned_lp = r.forward("default", data, None)["logprobs"][0]
    assert max(abs(a - b) for a, b in zip(tuned_lp, base_lp)) > 0.1
    before = {n: t.clone() for n, t in r.engine.iter_full_tensors("master") if "lora" not in n}
    out = ws.WeightSyncHandler(r).sync(backend="file", directory=str(tmp_path / "w"))
    assert out["synced"]
    for n, t in r.engine.iter_full_tensors("master"):
        if "lora" not in n:
            assert torch.equal(t, before[n]), n                      # folding happened on copies
    got = {}
    for f in sorted(os.listdir(tmp_path / "w")):
        if f.endswith(".safetensors"):
            got.update(load_file(str(tmp_path / "w" / f)))
    assert not any("lora" in k for k in got)
    # a plain model (no adapters) loaded from the same stream in fp32 (the bf16 rounding of the wire format
    # can flip a router's choice in a tiny random model, which says nothing about the folding)
    from xorl_b200.adapters.lora import merged_weight_view
    exact = dict(ws.iter_sync_tensors(r.engine, r.model.config, torch.float32, None, merged_weight_view(r.engine)))
    assert set(exact) == set(got)
    got = exact
    reset_parallel_state()
    sb = ServerArguments(model_preset=preset_name, output_dir=str(tmp_path / "srv2"), device="cpu",
                         sample_packing_sequence_len=256, enable_mixed_precision=False)
    r2 = ModelRunner(Trainer(sb.to_trainer_arguments()))
    from xorl_b200.checkpoint.handlers import get_checkpoint_handler
    from xorl_b200.checkpoint.hf_io import load_hf_weights
    from safetensors.torch import save_file
    os.makedirs(tmp_path / "hf")
    save_file({k: v.contiguous() for k, v in got.items()}, str(tmp_path / "hf" / "model.safetensors"))
    load_hf_weights(r2.engine, str(tmp_path / "hf"), r2.model.config)
    plain_lp = r2.forward("default", data, None)["logprobs"][0]
    moved = max(abs(a - b) for a, b in zip(tuned_lp, base_lp))
    off = max(abs(a - b) for a, b in zip(plain_lp, tuned_lp))
    assert off < 1e-4 and moved > 0.1, (off, moved)
    reset_parallel_state()


def test_fake_quantised_policy_syncs_its_wrapped_weights_on_the_trained_grid(tmp_path):
    """A server started with ``enable_qarl``: calibration ran at start-up, and a weight sync carries e4m3
    bytes + block scales for exactly the wrapped projections (not for the excluded one, the lm-head or the
    embedding), with the quantisation block the receiver needs."""
    import json
    from safetensors.torch import load_file
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server import weight_sync as ws
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    calib = tmp_path / "calib.json"
    calib.write_text(json.dumps({"input_ids": [list(range(3, 40)), list(range(9, 46))]}))
    with pytest.raises(ValueError):
        ServerArguments(model_preset="tiny-qwen3", enable_qarl=True, enable_lora=True)
    sa = ServerArguments(model_preset="tiny-qwen3", output_dir=str(tmp_path / "srv"), device="cpu",
                         sample_packing_sequence_len=256, enable_mixed_precision=False, enable_qarl=True,
                         qarl_exclude_modules=["down_proj"], qarl_calib_data=str(calib), qarl_calib_size=1)
    r = ModelRunner(Trainer(sa.to_trainer_arguments()))
    with open(tmp_path / "srv" / "qarl_calibration.json") as f:
        cal = json.load(f)
    assert cal["calibration_batches"] == 1 and cal["linear_count"] > 0
    out = ws.WeightSyncHandler(r).sync(backend="file", directory=str(tmp_path / "w"))
    assert out["quantization"] == "fp8" and out["quantization_config"]["weight_block_size"] == [128, 128]
    got = {}
    for f in sorted(os.listdir(tmp_path / "w")):
        if f.endswith(".safetensors"):
            got.update(load_file(str(tmp_path / "w" / f)))
    assert got["model.layers.0.mlp.up_proj.weight"].dtype == torch.uint8
    assert "model.layers.0.mlp.up_proj.weight_scale_inv" in got
    assert got["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16
    assert not any(k.startswith("lm_head") and k.endswith("scale_inv") for k in got)
    with pytest.raises(ValueError, match="differs"):
        ws.WeightSyncHandler(r).sync(backend="file", directory=str(tmp_path / "w2"), quantization="nvfp4")
    reset_parallel_state()


def test_endpoint_requests_revalidate_the_resolved_address(monkeypatch):
    """A hostname that resolved to a safe address at registration and to the metadata address
    later: the later request is refused, and requests go to the validated address literal, never
    to the hostname."""
    import socket
    from xorl_b200.server import weight_sync as ws
    answers = iter(["10.1.2.3", "10.1.2.3", "169.254.169.254"])
    seen = []

    def fake_getaddrinfo(host, port, *a, **k):
        ip = next(answers)
        seen.append((host, ip))
        return [(socket.AF_INET, socket.SOCK_STREAM, 6, "", (ip, port))]

    monkeypatch.setattr(socket, "getaddrinfo", fake_getaddrinfo)
    contacted = []
    em = ws.EndpointManager(post=lambda url, p: contacted.append(url) or {}, get=lambda url: {})
    info = em.add("http://engine.cluster.local:30000", 1)
    assert (info["host"], info["port"]) == ("engine.cluster.local", 30000)
    em.broadcast_post("/pause_generation", lambda e, off: {})
    assert contacted == ["http://10.1.2.3:30000/pause_generation"]        # the literal, not the name
    with pytest.raises(ValueError, match="unsafe endpoint address"):
        em.broadcast_post("/update_weights_from_distributed", lambda e, off: {})
    assert len(contacted) == 1 and [ip for _, ip in seen][-1] == "169.254.169.254"
    with pytest.raises(ValueError):
        em.add("http://engine.cluster.local:30000/some/path")
    with pytest.raises(ValueError):
        em.add("https://engine.cluster.local:30000")


def test_endpoint_manager_and_broadcast_group(tmp_path):
    from xorl_b200.server import weight_sync as ws
    calls = []
    em = ws.EndpointManager(post=lambda url, p: calls.append((url, p)) or {}, get=lambda url: {"ok": True},
                            url_of=lambda h, p, path: f"http://{h}:{p}{path}")
    em.add("http://a:1/", 2)
    em.add("http://b:1", 1)
    assert em.total_world() == 3 and em.check_health() == {"http://a:1": True, "http://b:1": True}
    em.broadcast_post("/init_weights_update_group", lambda e, off: {"rank_offset": off})
    assert [p["rank_offset"] for _, p in calls] == [1, 3]
    # a stateless 2-rank gloo group: trainer thread broadcasts a bucket, "engine" thread receives it
    from dist_utils import free_port
    port = free_port()
    bucket = [("w", torch.randn(4, 8).bfloat16())]
    flat, man = ws.flatten_bucket(bucket)
    got = {}

    def engine():
        g = ws.StatelessGroupBroadcaster("127.0.0.1", port, 1, 2, "gloo")
        got.update(g.recv_bucket(man, "cpu"))

    t = threading.Thread(target=engine)
    t.start()
    g0 = ws.StatelessGroupBroadcaster("127.0.0.1", port, 0, 2, "gloo")
    g0.send_bucket(bucket)
    t.join(30)
    assert torch.equal(got["w"], bucket[0][1])


def test_remote_backend_over_zmq():
    from xorl_b200.server.launcher import RemoteBackend, serve_zmq
    from dist_utils import free_port
    addr = f"tcp://127.0.0.1:{free_port()}"
    stop = threading.Event()
    be = DummyBackend()
    t = threading.Thread(target=serve_zmq, args=(be, addr, stop), daemon=True)
    t.start()
    rb = RemoteBackend(addr, timeout_ms=5000)
    out = rb.forward_backward("default", [{"tokens": [1, 2, 3]}], [[[0]]], "cross_entropy", {})
    assert out["num_tokens"] == 3 and rb.optim_step("default")["metrics"]["step"] == 1.0
    assert rb.health()["status"] == "ok"
    with pytest.raises(RuntimeError):
        rb._call("no_such_op", "default", {})
    stop.set()
    t.join(5)


def test_delta_codec_edge_cases():
    from xorl_b200.server.weight_sync import delta_apply, delta_encode
    a = torch.zeros(1000, dtype=torch.bfloat16)
    assert delta_apply(a.clone(), delta_encode(a, a)) == 0
    b = torch.ones(1000, dtype=torch.bfloat16)
    c = a.clone()
    assert delta_apply(c, delta_encode(a, b)) == 1000 and torch.equal(c, b)
    with pytest.raises(ValueError):
        delta_apply(torch.zeros(10, dtype=torch.bfloat16), delta_encode(a, b))


@pytest.mark.distributed
def test_dispatcher_two_ranks_agree_on_errors(tmp_path):
    from dist_utils import run_distributed
    out = run_distributed(os.path.join(os.path.dirname(__file__), "server_dispatch_worker.py"), 2, str(tmp_path))
    assert "DISPATCH_OK" in out


@pytest.mark.distributed
def test_adapter_replicas_are_compared_after_optimizer_steps(tmp_path):
    from dist_utils import run_distributed
    out = run_distributed(os.path.join(os.path.dirname(__file__), "server_replica_check_worker.py"), 2, str(tmp_path))
    assert "REPLICA_CHECK_OK" in out


@pytest.mark.distributed
def test_routing_replay_travels_beside_the_broadcast_command(tmp_path):
    from dist_utils import run_distributed
    out = run_distributed(os.path.join(os.path.dirname(__file__), "server_routing_payload_worker.py"), 2, str(tmp_path))
    assert "ROUTING_PAYLOAD_OK" in out


def test_routing_payload_chunks_and_checks(tmp_path):
    import base64
    import numpy as np
    from xorl_b200.server.side_payloads import (FilesystemPayloadStore, PayloadError, RoutingPayloads,
                                                canonical_routing, is_routing_ref)
    rp = RoutingPayloads(FilesystemPayloadStore(str(tmp_path / "p")), chunk_bytes=1000, min_bytes=0)
    g = torch.Generator().manual_seed(0)
    rows = [torch.randint(-1, 64, (n, 3, 4), generator=g) for n in (20, 7, 33)]
    enc = np.asarray(rows[1].numpy(), dtype="<i4")
    datums = [{"tokens": [1] * 20, "routed_experts": rows[0].tolist()},
              {"tokens": [1] * 7, "routed_experts": {"data": base64.b64encode(enc.tobytes()).decode(), "shape": [7, 3, 4],
                                                     "dtype": "int32"}},
              {"tokens": [1] * 5},
              {"tokens": [1] * 33, "routed_experts": rows[2]}]
    out, keys = rp.stash(datums)
    assert len(keys) == 2 and "routed_experts" not in out[2] and datums[0]["routed_experts"] == rows[0].tolist()
    for d, want in zip((out[0], out[1], out[3]), rows):
        assert is_routing_ref(d["routed_experts"]) and torch.equal(rp.resolve(d)["routed_experts"], want)
    # rows that do not match their checksum, rows that are gone
    ref = dict(out[0]["routed_experts"], offset=2)
    with pytest.raises(PayloadError, match="do not match"):
        rp.load(ref)
    assert rp.cleanup(keys)["chunks_deleted"] == 2 and rp.cleanup(keys)["chunks_deleted"] == 0
    with pytest.raises(PayloadError, match="gone"):
        rp.load(out[0]["routed_experts"])
    with pytest.raises(PayloadError):
        canonical_routing(torch.full((2, 1, 1), 40000))
    small = RoutingPayloads(FilesystemPayloadStore(str(tmp_path / "q")))       # default threshold: tiny requests stay inline
    same, none = small.stash(datums)
    assert same is datums and none == []


def _lora_runner(tmp_path, preset="tiny-qwen3"):
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    sa = ServerArguments(model_preset=preset, output_dir=str(tmp_path / "srv"), device="cpu",
                         sample_packing_sequence_len=256, enable_mixed_precision=False, enable_lora=True,
                         lora_rank=4, lora_alpha=8)
    return ModelRunner(Trainer(sa.to_trainer_arguments()))


def test_multi_tenant_adapters_are_isolated(tmp_path):
    os.environ["XORL_MAX_ADAPTERS_PER_MODEL"] = "2"
    try:
        r = _lora_runner(tmp_path)
        data = [{"tokens": list(range(3, 60))}]

        def lp(mid):
            return r.forward(mid, data, None)["logprobs"][0]

        def train(mid, steps):
            for _ in range(steps):
                r.forward_backward(mid, data, None)
                r.optim_step(mid, adam_params={"learning_rate": 5e-3})

        base = lp("default")
        r.create_model("a")
        r.create_model("b")
        assert lp("a") == base and lp("b") == base            # fresh adapters start as the base model
        train("a", 3)
        la = lp("a")
        assert max(abs(x - y) for x, y in zip(la, base)) > 1e-3
        assert lp("b") == base and lp("default") == base      # a's training moved nothing else
        train("b", 2)
        assert lp("a") == la                                   # ... and b's training did not move a
        # reference pass: the frozen base model's log-probabilities, whatever the adapter has learned
        ref = r.forward("a", data, None, loss_fn_config={"reference": True})["logprobs"][0]
        assert ref == base and lp("a") == la                   # and the adapter is back in place afterwards
        # an open gradient epoch survives a switch to another adapter and back
        r.forward_backward("a", data, None)
        tokens_a = r.accumulated_tokens
        r.forward_backward("b", data, None)
        r.abort_gradient_epoch("b")
        m = r.optim_step("a", adam_params={"learning_rate": 5e-3})["metrics"]
        assert m["tokens"] == tokens_a and m["step"] == 4.0
        # three adapters with a cap of two in memory: the least recently used one went to disk and comes back
        assert os.path.isdir(os.path.join(r.output_dir, "adapter_spill"))
        assert lp("default") == base
        r.unload_model("b")
        with pytest.raises(KeyError):
            r.forward("b", data, None)
    finally:
        del os.environ["XORL_MAX_ADAPTERS_PER_MODEL"]
        from xorl_b200.parallel.state import reset_parallel_state
        reset_parallel_state()


def test_adapter_sessions_have_their_own_rank_alpha_and_learning_rate(tmp_path):
    """A session of rank 2 in a server of capacity 4: its rank components 2 and 3 start at zero and stay
    zero through training (so it is a rank-2 adapter), its scale is its own alpha / rank, and the
    learning rate it was last stepped with stays with it across switches."""
    import torch
    r = _lora_runner(tmp_path)
    data = [{"tokens": list(range(3, 60))}]
    out = r.create_model("small", lora_config={"rank": 2, "alpha": 6})
    assert out["session"]["rank"] == 2 and out["session"]["alpha"] == 6
    with pytest.raises(ValueError):
        r.create_model("too_big", lora_config={"rank": 8})
    assert "too_big" not in r.adapters.list()
    for _ in range(3):
        r.forward_backward("small", data, None)
        r.optim_step("small", adam_params={"learning_rate": 7e-3})
    from xorl_b200.adapters.lora import LoraLinear
    mods = [m for m in r.engine.model.modules() if isinstance(m, LoraLinear)]
    assert mods and all(m.scaling == 3.0 for m in mods)
    full = dict(r.engine.iter_full_tensors("master"))
    moved = 0
    for n, t in full.items():
        if "lora_A" in n:
            assert float(t[2:].abs().max()) == 0.0 and float(t[:2].abs().max()) > 0, n
        if "lora_B" in n:
            assert float(t[:, 2:].abs().max()) == 0.0, n
            moved += float(t[:, :2].abs().max()) > 0
    assert moved > 0
    # back on the default adapter: the server's alpha / rank and learning rate; the session keeps its own
    r.forward_backward("default", data, None)
    r.optim_step("default", adam_params={"learning_rate": 1e-3})
    assert all(m.scaling == 2.0 for m in mods)
    assert r.adapters.get_lr("small") == 7e-3 and r.adapters.get_lr("default") == 1e-3
    r.adapters.set_lr("small", 2e-3)
    r.forward_backward("small", data, None)
    assert r.optim_step("small")["metrics"]["learning_rate"] == 2e-3
    usage = r.adapters.memory_usage()
    assert set(usage) == {"default", "small"} and all(v > 0 for v in usage.values())
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()


def test_sampler_weights_of_a_lora_session_are_its_adapter_at_its_own_rank(tmp_path):
    """``save_sampler_weights`` on a LoRA server writes a PEFT directory for the session (rank 2 of the
    server's 4: matrices cut to two components, ``r`` / ``lora_alpha`` the session's), refuses a name that
    exists, and with ``merged`` writes full weights instead."""
    import json
    from safetensors.torch import load_file
    r = _lora_runner(tmp_path)
    data = [{"tokens": list(range(3, 60))}]
    r.create_model("small", lora_config={"rank": 2, "alpha": 6})
    r.forward_backward("small", data, None)
    r.optim_step("small", adam_params={"learning_rate": 5e-3})
    out = r.save_sampler_weights("small", "s1")
    assert out["kind"] == "lora_adapter"
    cfg = json.load(open(os.path.join(out["directory"], "adapter_config.json")))
    assert cfg["r"] == 2 and cfg["lora_alpha"] == 6 and cfg["peft_type"] == "LORA"
    t = load_file(os.path.join(out["directory"], "adapter_model.safetensors"))
    a = [v for k, v in t.items() if "lora_A" in k]
    b = [v for k, v in t.items() if "lora_B" in k]
    assert a and all(v.shape[0] == 2 for v in a) and all(v.shape[1] == 2 for v in b)
    assert any(float(v.abs().max()) > 0 for v in b)
    with pytest.raises(ValueError, match="exist"):
        r.save_sampler_weights("small", "s1")
    full = r.save_sampler_weights("default", "s2")
    assert json.load(open(os.path.join(full["directory"], "adapter_config.json")))["r"] == 4
    merged = r.save_sampler_weights("small", "s3", merged=True)
    assert merged["kind"] == "full_weights" and merged["synced"]
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()


def test_saves_are_refused_beyond_the_storage_limit(tmp_path):
    from fastapi.testclient import TestClient
    from xorl_b200.server.api_server import ServerState, create_app
    from xorl_b200.server.backend import DummyBackend
    out = tmp_path / "o"
    os.makedirs(out / "sampler_weights" / "taken")
    (out / "blob.bin").write_bytes(b"x" * 4096)
    st = ServerState(DummyBackend(), str(out), storage_limit_bytes=1024)
    with TestClient(create_app(st)) as c:
        assert c.post("/api/v1/save_weights", json={"path": "a"}).status_code == 507
        assert c.post("/api/v1/save_weights_for_sampler", json={"path": "b"}).status_code == 507
        st.storage_limit_bytes = 0
        assert c.post("/api/v1/save_weights_for_sampler", json={"path": "taken"}).status_code == 409
        rid = c.post("/api/v1/save_weights_for_sampler", json={"path": "fresh"}).json()["request_id"]
        assert _poll(c, rid)["type"] == "save_weights_for_sampler"


def test_server_arguments_reach_the_runner(tmp_path):
    """``max_adapters_per_model``, ``enable_moe_metrics`` and ``sync_bucket_size_mb`` of the server configuration
    are what the runner works with."""
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server.launcher import build_local_backend
    from xorl_b200.server.server_arguments import ServerArguments
    reset_parallel_state()
    sa = ServerArguments(model_preset="tiny-qwen3-moe", output_dir=str(tmp_path / "srv"), device="cpu",
                         sample_packing_sequence_len=256, enable_mixed_precision=False, enable_lora=True, lora_rank=4,
                         max_adapters_per_model=2, enable_moe_metrics=False, sync_bucket_size_mb=1)
    backend, _ = build_local_backend(sa)
    r = backend.runner
    assert r.moe_metrics is None
    r.create_model("a")
    assert r.adapters.max_adapters == 2
    out = r.sync_inference_weights("default", backend="file", directory=str(tmp_path / "w"))
    assert out["buckets"] > 1                                   # one-megabyte buckets, not the 1 GiB default
    out = r.sync_inference_weights("default", backend="file", directory=str(tmp_path / "w2"), bucket_size_mb=1024)
    assert out["buckets"] == 1
    reset_parallel_state()


def test_adapter_with_pending_gradients_is_not_dropped(tmp_path):
    """Without a spill directory an adapter that holds accumulated gradients is never the eviction
    victim; when every resident adapter holds some, creating another one raises."""
    os.environ["XORL_MAX_ADAPTERS_PER_MODEL"] = "3"
    try:
        r = _lora_runner(tmp_path)
        data = [{"tokens": list(range(3, 60))}]
        r.create_model("a")
        r.adapters.spill_dir = None
        r.create_model("b")
        r.forward_backward("a", data, None)                    # a: open epoch
        r.forward_backward("b", data, None)                    # b: open epoch (a now rests on the host)
        r.forward_backward("default", data, None)              # default active; a and b resident
        with pytest.raises(RuntimeError, match="accumulated gradients"):
            r.create_model("c")
        assert "c" not in r.adapters.list()
        r.optim_step("a", adam_params={"learning_rate": 1e-3})  # a is clean now (and active)
        r.forward_backward("default", data, None)              # default active again: a rests clean, b pending
        r.create_model("c")                                    # evicts a, the only clean resident one
        assert sorted(r.adapters.list()) == ["b", "c", "default"]
        assert r.optim_step("b", adam_params={"learning_rate": 1e-3})["metrics"]["tokens"] > 0
    finally:
        del os.environ["XORL_MAX_ADAPTERS_PER_MODEL"]
        from xorl_b200.parallel.state import reset_parallel_state
        reset_parallel_state()


def test_rollout_routing_replay(tmp_path):
    from xorl_b200.parallel.state import reset_parallel_state
    from xorl_b200.server.runner import ModelRunner
    from xorl_b200.server.server_arguments import ServerArguments
    from xorl_b200.trainers.trainer import Trainer
    reset_parallel_state()
    sa = ServerArguments(model_preset="tiny-qwen3-moe", output_dir=str(tmp_path / "srv"), device="cpu",
                         sample_packing_sequence_len=128, enable_mixed_precision=False)
    r = ModelRunner(Trainer(sa.to_trainer_arguments()))
    toks = list(range(5, 45))
    free = r.forward_backward("default", [{"tokens": toks}], None)["loss"]
    r.abort_gradient_epoch()
    # force every token of both MoE layers to experts (0, 1): a different (worse or equal) loss, and
    # the load statistics must show only those two experts
    forced = [[[0, 1], [0, 1]] for _ in toks]
    loads = []
    orig_add = r.moe_metrics.add
    r.moe_metrics.add = lambda layer, counts: (loads.append(counts.clone()), orig_add(layer, counts))[1]
    out = r.forward_backward("default", [{"tokens": toks, "routed_experts": forced}], None)
    assert out["metrics"]["moe/max_imbalance_ratio"] > 1.5          # two experts took (almost) everything
    import json as _json
    rec = [_json.loads(l) for l in open(os.path.join(r.output_dir, "moe_metrics.jsonl"))][-1]
    assert rec["expert_load"]["num_moe_layers"] == len(loads) and rec["expert_load"]["total_tokens"] == 2 * 128 * len(loads)
    pad = 128 - len(toks)                                   # padding rows keep the router's own choice
    assert loads and all(int(l[0]) >= len(toks) and int(l[1]) >= len(toks) and int(l[2:].sum()) <= 2 * pad
                         for l in loads)
    assert abs(out["loss"] - free) > 1e-6
    reset_parallel_state()
