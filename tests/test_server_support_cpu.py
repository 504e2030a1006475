"""Server support modules: security boundaries, session specs, side payload store."""
import os

import pytest
import torch


def test_identifiers_and_confined_paths(tmp_path):
    from xorl_b200.server.security import artifact_path, confine_path, validate_identifier
    assert validate_identifier("run-01.step_5") == "run-01.step_5"
    for bad in ("", "..", "../x", "a/b", ".hidden", "x" * 200, "a b"):
        with pytest.raises(ValueError):
            validate_identifier(bad)
    root = tmp_path / "out"
    (root / "ckpt").mkdir(parents=True)
    assert confine_path(root, "ckpt/a.pt") == (root / "ckpt" / "a.pt").resolve()
    for bad in ("../secret", "/etc/passwd", "ckpt/../../x"):
        with pytest.raises(ValueError):
            confine_path(root, bad)
    os.symlink("/etc", root / "link")
    with pytest.raises(ValueError):
        confine_path(root, "link/passwd")
    with pytest.raises(FileNotFoundError):
        confine_path(root, "ckpt/missing", must_exist=True)
    with pytest.raises(ValueError):
        artifact_path("  ", root=root)
    assert artifact_path("ckpt", root=root, must_exist=True).name == "ckpt"


def test_outbound_endpoints(monkeypatch):
    from xorl_b200.server.security import ALLOWLIST_ENV, endpoint_url, validate_endpoint
    monkeypatch.delenv(ALLOWLIST_ENV, raising=False)
    assert validate_endpoint("127.0.0.1", 30000) == ("127.0.0.1", 30000)
    assert endpoint_url("127.0.0.1", "8000", "/health", require_allowlist=True) == "http://127.0.0.1:8000/health"
    assert endpoint_url("::1", 8000, "/health") == "http://[::1]:8000/health"
    for host, port in (("169.254.169.254", 80), ("0.0.0.0", 80), ("224.0.0.1", 80), ("a/b", 80), ("h@x", 80),
                       ("10.0.0.1", 0), ("10.0.0.1", 70000), ("bad host", 80)):
        with pytest.raises(ValueError):
            validate_endpoint(host, port)
    with pytest.raises(ValueError):
        validate_endpoint("10.1.2.3", 8000, require_allowlist=True)          # no allow-list configured
    monkeypatch.setenv(ALLOWLIST_ENV, "10.1.0.0/16, engine.internal")
    assert validate_endpoint("10.1.2.3", 8000, require_allowlist=True) == ("10.1.2.3", 8000)
    with pytest.raises(ValueError):
        validate_endpoint("10.2.0.1", 8000, require_allowlist=True)
    with pytest.raises(ValueError):
        endpoint_url("127.0.0.1", 80, "/x?y=1")


def test_session_spec_roundtrip(tmp_path):
    from xorl_b200.server.session_spec import (normalize_session_spec, optimizer_build_kwargs, read_session_spec,
                                               write_session_spec)
    defaults = dict(default_rank=16, default_alpha=32, max_rank=64, server_targets=["qkv_proj", "o_proj"])
    spec = normalize_session_spec(base_model="Qwen/Qwen3-8B", lora={"r": 8, "lora_alpha": 16, "target_modules": ["o_proj"]},
                                  optimizer={"type": "AdamW", "lr": 3e-5, "betas": [0.9, 0.99]}, lora_defaults=defaults)
    assert spec["lora"] == {"rank": 8, "alpha": 16.0, "target_modules": ["o_proj"], "dropout": 0.0}
    assert spec["optimizer"]["type"] == "adamw" and spec["optimizer"]["eps"] == 1e-12
    kw = optimizer_build_kwargs(spec["optimizer"])
    assert kw["lr"] == 3e-5 and kw["betas"] == (0.9, 0.99) and kw["optimizer_type"] == "adamw"
    for bad in (dict(lora={"r": 128}), dict(lora={"rank": 8, "bogus": 1}), dict(lora={"target_modules": ["lm_head"]}),
                dict(optimizer={"type": "lion"}), dict(optimizer={"lr": float("nan")}), dict(optimizer={"betas": [1.0, 0.9]}),
                dict(optimizer={"momentum": 0.9})):
        with pytest.raises(ValueError):
            normalize_session_spec(base_model="m", lora=bad.get("lora"), optimizer=bad.get("optimizer"), lora_defaults=defaults)
    write_session_spec(str(tmp_path / "s"), spec)
    assert read_session_spec(str(tmp_path / "s")) == spec
    # an older checkpoint with only the PEFT adapter config
    old = tmp_path / "old"
    old.mkdir()
    (old / "adapter_config.json").write_text('{"r": 4, "lora_alpha": 8, "target_modules": ["qkv_proj"]}')
    got = read_session_spec(str(old), fallback=spec)
    assert got["lora"]["rank"] == 4 and got["lora"]["target_modules"] == ["qkv_proj"] and got["optimizer"] == spec["optimizer"]
    with pytest.raises(FileNotFoundError):
        read_session_spec(str(tmp_path / "none"))


def test_side_payload_store(tmp_path):
    from xorl_b200.server.side_payloads import FilesystemPayloadStore, PayloadError, is_payload_ref, resolve_refs
    store = FilesystemPayloadStore(str(tmp_path / "payloads"), ttl_seconds=10.0, max_bytes=1 << 20)
    routing = torch.randint(0, 128, (300, 4, 8), dtype=torch.int16)
    ref = store.put(routing)
    assert is_payload_ref(ref) and ref["nbytes"] > routing.numel() * 2
    req = {"datum": {"tokens": [1, 2, 3], "routing": ref}, "other": [ref, 5]}
    out = resolve_refs(req, store)
    assert torch.equal(out["datum"]["routing"], routing) and torch.equal(out["other"][0], routing) and out["other"][1] == 5
    with pytest.raises(PayloadError):
        store.get({**ref, "sha256": "0" * 64})
    with pytest.raises(PayloadError):
        store.put(torch.zeros(1 << 20))                                  # over the size limit
    with pytest.raises(ValueError):
        store.get({**ref, "key": "../escape"})
    assert store.sweep(now=os.path.getmtime(tmp_path / "payloads" / (ref["key"] + ".pt")) + 5) == 0
    assert store.sweep(now=os.path.getmtime(tmp_path / "payloads" / (ref["key"] + ".pt")) + 11) == 1
    with pytest.raises(PayloadError):
        store.get(ref)


def test_r3_staging_benchmark_runs(capsys):
    from xorl_b200.utils.r3_staging_bench import main
    out = main(["--datums", "6", "--tokens", "128", "--layers", "3", "--top-k", "2", "--pack-len", "512"])
    assert out["micro_batches"] >= 2 and out["payload_mb"] > 0 and out["store_put_s"] > 0


def test_supervisor_tears_the_service_down_when_a_member_dies(tmp_path):
    """Two children; one exits with code 3: the other (which ignores nothing) is terminated, the
    whole process group with it, and the supervisor returns 3."""
    import sys
    import time
    from xorl_b200.server.supervisor import ChildSpec, Supervisor
    marker = tmp_path / "ready"
    sleeper = [sys.executable, "-c", "import time, subprocess, sys\n"
               "p = subprocess.Popen([sys.executable, '-c', 'import time; time.sleep(600)'])\n"
               f"open({str(marker)!r}, 'w').write(str(p.pid))\ntime.sleep(600)"]
    dier = [sys.executable, "-c", "import time, sys; time.sleep(1.5); sys.exit(3)"]
    sup = Supervisor([ChildSpec("workers", sleeper, ready=lambda: marker.exists()),
                      ChildSpec("api", dier)], poll_interval=0.05, grace=3.0, log=lambda m: None)
    t0 = time.time()
    assert sup.run(install_signal_handlers=False) == 3
    assert time.time() - t0 < 15 and sup.first_exit == "api"
    assert any("workers ready" in e for e in sup.events)
    for c in sup.children:
        assert c.proc.poll() is not None
    grandchild = int(marker.read_text())
    time.sleep(0.3)
    try:                                   # the worker's own child (same process group) is gone too
        os.kill(grandchild, 0)
        alive = os.path.exists(f"/proc/{grandchild}") and "Z" not in open(f"/proc/{grandchild}/stat").read().split()[2]
    except ProcessLookupError:
        alive = False
    assert not alive


def test_supervisor_stops_on_request_and_on_unanswered_probes(tmp_path):
    import sys
    import threading
    import time
    from xorl_b200.server.supervisor import ChildSpec, Supervisor
    sleeper = [sys.executable, "-c", "import time; time.sleep(600)"]
    # a member that never becomes ready
    sup = Supervisor([ChildSpec("workers", sleeper, ready=lambda: False, ready_timeout=1.0)],
                     poll_interval=0.05, grace=2.0, log=lambda m: None)
    assert sup.run(install_signal_handlers=False) == 1 and sup.children[0].proc.poll() is not None
    # a member whose liveness probe stops answering
    state = {"ok": True}
    sup = Supervisor([ChildSpec("api", sleeper, alive=lambda: state["ok"])], poll_interval=0.05, grace=2.0,
                     liveness_timeout=0.5, log=lambda m: None)
    threading.Timer(0.7, lambda: state.update(ok=False)).start()
    assert sup.run(install_signal_handlers=False) == 1
    assert any("unresponsive" in e for e in sup.events)
    # an orderly stop request
    sup = Supervisor([ChildSpec("api", sleeper)], poll_interval=0.05, grace=2.0, log=lambda m: None)
    threading.Timer(0.5, sup.request_stop).start()
    assert sup.run(install_signal_handlers=False) == 0 and sup.children[0].proc.poll() is not None


@pytest.mark.distributed
def test_weight_sync_stream_covers_all_pipeline_stages(tmp_path):
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_distributed
    out = run_distributed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "weight_sync_pp_worker.py"), 2,
                          str(tmp_path / "o"))
    assert "PP_SYNC_OK" in out


@pytest.mark.distributed
def test_service_runner_under_pipeline_parallelism(tmp_path):
    import json
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from dist_utils import run_distributed
    from server_pp_worker import build_runner, drive
    from xorl_b200.parallel.state import reset_parallel_state
    reset_parallel_state()
    ref = drive(build_runner(str(tmp_path / "ref"), pp=1))
    reset_parallel_state()
    ref_path = tmp_path / "ref.json"
    ref_path.write_text(json.dumps(ref))
    out = run_distributed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "server_pp_worker.py"), 2,
                          str(tmp_path / "pp"), str(ref_path))
    assert "PP_RUNNER_OK" in out


def test_server_arguments_reject_inconsistent_settings():
    from xorl_b200.server.server_arguments import ServerArguments
    ServerArguments(sample_packing_strategy="balanced_dp", sample_packing_on_oversized="truncate")
    for kw, msg in ((dict(sample_packing_strategy="tetris"), "sample_packing_strategy"),
                    (dict(sample_packing_on_oversized="drop"), "on_oversized"),
                    (dict(pipeline_parallel_size=0), "pipeline_parallel_size"),
                    (dict(api_port=70000), "api_port"),
                    (dict(enable_qlora=True), "enable_qlora"),
                    (dict(worker_bind_address="127.0.0.1:5555"), "worker_bind_address")):
        with pytest.raises(ValueError, match=msg):
            ServerArguments(**kw)


def test_every_server_argument_is_read_somewhere():
    """No key of the service configuration is accepted and then ignored: each is read outside its own
    declaration (by the launcher, the API state, the runner) or mapped into the trainer's arguments."""
    import dataclasses
    import glob
    import re
    from xorl_b200.server.server_arguments import ServerArguments
    root = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "xorl_b200")
    own = open(os.path.join(root, "server", "server_arguments.py")).read()
    src = "".join(open(f).read() for f in glob.glob(os.path.join(root, "**", "*.py"), recursive=True))
    mapped = own.split("def to_trainer_arguments")[1]
    unused = []
    for f in dataclasses.fields(ServerArguments):
        elsewhere = len(re.findall(r"\.%s\b" % f.name, src)) - len(re.findall(r"self\.%s\b" % f.name, own))
        if elsewhere <= 0 and not re.search(r"self\.%s\b" % f.name, mapped):
            unused.append(f.name)
    assert not unused, unused
