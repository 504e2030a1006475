"""Starts the training service.

``--mode launch`` starts the worker fleet (torchrun) and the API process as children of a supervisor
(``server/supervisor.py``) that tears the service down when a member dies.
``--mode auto`` builds the worker in this process group: under ``torchrun`` every rank builds the
trainer; rank 0 additionally runs the REST server with a backend that broadcasts each command to
the other ranks, which sit in ``RunnerDispatcher.worker_loop``.  ``--mode connect`` starts only the
API process and talks to an already running worker fleet over ZMQ (``RemoteBackend``); the fleet's
rank 0 runs ``serve_zmq`` (src/xorl/server/launcher.py:160-1153, backend/remote.py).
"""
from __future__ import annotations

import argparse
import os
import threading
from typing import Any, Dict, Optional

import torch.distributed as dist

from .api_server import ServerState, create_app
from .backend import Backend, LocalBackend
from .runner import ModelRunner, RunnerDispatcher
from .server_arguments import ServerArguments

_OPS = ("forward_backward", "forward", "optim_step", "save_weights", "load_weights",
        "sync_inference_weights", "save_sampler_weights", "abort_gradient_epoch", "sleep", "wake_up", "create_model", "unload_model")


class DispatchBackend(Backend):
    """Backend of rank 0 in a multi-rank fleet: every call becomes a broadcast command."""

    def __init__(self, dispatcher: RunnerDispatcher):
        self.d = dispatcher
        self._lock = threading.Lock()
        # large routing-replay tensors travel beside the broadcast command, not inside it
        self.payloads = getattr(dispatcher.runner, "payloads", None)

    def _call(self, op: str, model_id: str, args: Dict[str, Any]):
        with self._lock:
            out = self.d.execute({"op": op, "model_id": model_id, "args": args})
        if "error" in out and out["error"]:
            raise RuntimeError(out["error"])
        return out["result"]

    def _with_payloads(self, op, model_id, datums, plan, loss_fn, loss_fn_config):
        keys = []
        if self.payloads is not None:
            datums, keys = self.payloads.stash(datums)
        try:
            return self._call(op, model_id, dict(datums=datums, plan=plan, loss_fn=loss_fn,
                                                 loss_fn_config=loss_fn_config))
        finally:
            if keys:
                self.payloads.cleanup(keys)          # every rank has answered (or failed together) by now

    def forward_backward(self, model_id, datums, plan, loss_fn, loss_fn_config):
        return self._with_payloads("forward_backward", model_id, datums, plan, loss_fn, loss_fn_config)

    def forward(self, model_id, datums, plan, loss_fn, loss_fn_config):
        return self._with_payloads("forward", model_id, datums, plan, loss_fn, loss_fn_config)

    def optim_step(self, model_id, **kw):
        return self._call("optim_step", model_id, kw)

    def save_weights(self, model_id, **kw):
        return self._call("save_weights", model_id, kw)

    def load_weights(self, model_id, **kw):
        return self._call("load_weights", model_id, kw)

    def sync_inference_weights(self, model_id, **kw):
        return self._call("sync_inference_weights", model_id, kw)

    def save_sampler_weights(self, model_id, **kw):
        return self._call("save_sampler_weights", model_id, kw)

    def abort_gradient_epoch(self, model_id, **kw):
        return self._call("abort_gradient_epoch", model_id, {})

    def create_model(self, model_id, **kw):
        return self._call("create_model", model_id, kw)

    def unload_model(self, model_id, **kw):
        return self._call("unload_model", model_id, kw)

    def shutdown(self):
        with self._lock:
            self.d.execute({"op": "shutdown"})


class RemoteBackend(Backend):
    """REQ/REP client of a worker fleet (msgpack frames over ZMQ)."""

    def __init__(self, address: str, timeout_ms: int = 600_000):
        import zmq
        self.ctx = zmq.Context.instance()
        self.address, self.timeout_ms = address, timeout_ms
        self._lock = threading.Lock()
        self._connect()

    def _connect(self):
        import zmq
        self.sock = self.ctx.socket(zmq.REQ)
        self.sock.setsockopt(zmq.RCVTIMEO, self.timeout_ms)
        self.sock.setsockopt(zmq.LINGER, 0)
        self.sock.connect(self.address)

    def _call(self, op, model_id, args):
        import msgpack
        import zmq
        with self._lock:
            self.sock.send(msgpack.packb({"op": op, "model_id": model_id, "args": args}, use_bin_type=True))
            try:
                out = msgpack.unpackb(self.sock.recv(), raw=False)
            except zmq.Again:
                self.sock.close()
                self._connect()          # a REQ socket cannot be reused after a lost reply
                raise TimeoutError(f"worker fleet did not answer {op} within {self.timeout_ms} ms")
        if out.get("error"):
            raise RuntimeError(out["error"])
        return out.get("result")

    def health(self):
        try:
            return self._call("health", "default", {})
        except Exception as e:  # noqa: BLE001
            return {"status": "unreachable", "error": str(e)}


for _op in _OPS:
    if _op in ("forward_backward", "forward"):
        def _m(self, model_id, datums, plan, loss_fn, loss_fn_config, _op=_op):
            return self._call(_op, model_id, dict(datums=datums, plan=plan, loss_fn=loss_fn,
                                                  loss_fn_config=loss_fn_config))
    else:
        def _m(self, model_id="default", _op=_op, **kw):
            return self._call(_op, model_id, kw)
    setattr(RemoteBackend, _op, _m)


def serve_zmq(backend: Backend, address: str, stop: Optional[threading.Event] = None) -> None:
    """Worker-side loop for ``RemoteBackend`` clients."""
    import msgpack
    import zmq
    ctx = zmq.Context.instance()
    sock = ctx.socket(zmq.REP)
    sock.setsockopt(zmq.RCVTIMEO, 200)
    sock.setsockopt(zmq.LINGER, 0)
    sock.bind(address)
    try:
        while stop is None or not stop.is_set():
            try:
                msg = msgpack.unpackb(sock.recv(), raw=False)
            except zmq.Again:
                continue
            op = msg.get("op")
            try:
                if op == "health":
                    res = backend.health()
                elif op == "shutdown":
                    sock.send(msgpack.packb({"result": {"shutdown": True}}, use_bin_type=True))
                    return
                elif op in ("forward_backward", "forward"):
                    a = msg["args"]
                    res = getattr(backend, op)(msg["model_id"], a["datums"], a["plan"], a["loss_fn"],
                                               a["loss_fn_config"])
                elif op in _OPS:
                    res = getattr(backend, op)(msg["model_id"], **msg.get("args", {}))
                else:
                    raise ValueError(f"unknown op {op!r}")
                sock.send(msgpack.packb({"result": res}, use_bin_type=True))
            except Exception as e:  # noqa: BLE001
                sock.send(msgpack.packb({"error": f"{type(e).__name__}: {e}"}, use_bin_type=True))
    finally:
        sock.close()


def build_local_backend(sargs: ServerArguments):
    """Trainer + runner in this process (every rank calls this)."""
    from ..trainers.trainer import Trainer
    trainer = Trainer(sargs.to_trainer_arguments())
    runner = ModelRunner(trainer, max_adapters=sargs.max_adapters_per_model, moe_metrics=sargs.enable_moe_metrics,
                         sync_bucket_size_mb=sargs.sync_bucket_size_mb)
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        return LocalBackend(runner), None
    cpu_group = dist.new_group(backend="gloo")
    disp = RunnerDispatcher(runner, cpu_group)
    return (DispatchBackend(disp) if dist.get_rank() == 0 else None), disp


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(description="xorl_b200 training service")
    ap.add_argument("--mode", choices=["auto", "connect", "worker", "launch"], default="auto")
    ap.add_argument("--nproc", type=int, default=0,
                    help="--mode launch: ranks of the worker fleet (default: all visible GPUs, at least 1)")
    ap.add_argument("--master-port", type=int, default=29400)
    ap.add_argument("--config", required=True)
    ap.add_argument("--api-host", default=None)
    ap.add_argument("--api-port", type=int, default=None)
    ap.add_argument("--worker-address", default=None)
    ns = ap.parse_args(argv)
    sargs = ServerArguments.from_yaml(ns.config)
    if ns.api_host:
        sargs.api_host = ns.api_host
    if ns.api_port:
        sargs.api_port = ns.api_port
    if ns.worker_address:
        sargs.worker_bind_address = ns.worker_address

    if ns.mode == "launch":
        # separate processes under a supervisor: torchrun worker fleet + API process; when one of them
        # exits or stops answering, the other is torn down and the exit code is passed on
        import sys
        import torch
        from .supervisor import Supervisor, service_children
        nproc = ns.nproc or max(1, torch.cuda.device_count())
        sup = Supervisor(service_children(ns.config, nproc, sargs.api_host, sargs.api_port,
                                          sargs.worker_bind_address, ns.master_port))
        sys.exit(sup.run())
    if ns.mode == "connect":
        backend: Backend = RemoteBackend(sargs.worker_bind_address)
        dp = 1
    else:
        backend, disp = build_local_backend(sargs)
        if backend is None:            # non-zero ranks only execute broadcast commands
            disp.worker_loop()
            return
        from ..parallel.state import get_parallel_state
        dp = get_parallel_state().dp_size
        if ns.mode == "worker":
            serve_zmq(backend, sargs.worker_bind_address)
            if hasattr(backend, "shutdown"):
                backend.shutdown()
            return
    import uvicorn
    state = ServerState(backend, sargs.output_dir, dp, sargs.sample_packing_sequence_len,
                        sargs.sample_packing_strategy or sargs.sample_packing_method, sargs.future_ttl_seconds,
                        sargs.session_timeout_seconds, sargs.api_keys, sargs.idle_sleep_seconds,
                        on_oversized=sargs.sample_packing_on_oversized,
                        storage_limit_bytes=int(sargs.storage_limit_gb * (1 << 30)))
    try:
        uvicorn.run(create_app(state), host=sargs.api_host, port=sargs.api_port, log_level="info")
    finally:
        if hasattr(backend, "shutdown"):
            backend.shutdown()


if __name__ == "__main__":
    main()
