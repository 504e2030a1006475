"""REST front end of the training service (FastAPI).

Two-phase protocol: mutating calls return a request id at once, the orchestrator runs them in
order on the backend, and ``/api/v1/retrieve_future`` is polled for the outcome (``try_again``
while pending, the typed result when done, ``request_failed`` with a category on error)
(src/xorl/server/api_server/endpoints.py:192-1133, server.py).  Sessions expire without
heartbeats, which releases their models; an idle watchdog can release device memory when nobody
has called for a while.
"""
from __future__ import annotations

import contextlib
import os
import shutil
import threading
import time
import uuid
from typing import Any, Dict, List, Optional

from fastapi import Depends, FastAPI, Header, HTTPException

from . import api_types as T
from .future_store import FutureStore
from .orchestrator import Orchestrator, OrchestratorRequest, RequestProcessor, SeqIdAwareFIFOPolicy
from .security import validate_identifier
from .weight_sync import EndpointManager


def _datum_to_dict(d: T.Datum) -> Dict[str, Any]:
    out: Dict[str, Any] = {"tokens": d.model_input.token_ids()}
    for k, v in d.loss_fn_inputs.items():
        out[k] = v.to_list()
    return out


class ServerState:
    def __init__(self, backend, output_dir: str = "outputs", dp_size: int = 1, packing_len: int = 4096,
                 packing: str = "sequential", future_ttl: float = 3600.0, session_timeout: float = 600.0,
                 api_keys: Optional[List[str]] = None, idle_sleep_seconds: float = 0.0,
                 on_oversized: str = "error", storage_limit_bytes: int = 0):
        self.backend = backend
        self.output_dir = output_dir
        self.storage_limit_bytes = int(storage_limit_bytes)      # 0 = no limit on what is kept under output_dir
        self.futures = FutureStore(future_ttl)
        self.endpoints = EndpointManager()
        self.orch = Orchestrator(backend, SeqIdAwareFIFOPolicy(),
                                 RequestProcessor(dp_size, packing_len, packing, on_oversized=on_oversized),
                                 self._on_result)
        self.sessions: Dict[str, Dict[str, Any]] = {}
        self.models: Dict[str, Dict[str, Any]] = {"default": {"model_id": "default", "created": time.time()}}
        self.training_runs: Dict[str, Dict[str, Any]] = {}
        self.session_timeout = session_timeout
        self.api_keys = set(api_keys or [])
        self.sync_quantization: Optional[str] = None
        self.asleep = False
        self.last_activity = time.time()
        self.idle_sleep_seconds = idle_sleep_seconds
        self.started = time.time()
        self._lock = threading.Lock()
        self._post: Dict[str, Any] = {}

    # ---- futures ---------------------------------------------------------------------------
    def _on_result(self, rid: str, res: Any, err: Optional[str]) -> None:
        if err is not None:
            cat = "user" if err.startswith(("ValueError", "KeyError")) else "server"
            self.futures.set_error(rid, err, cat)
            return
        hook = self._post.pop(rid, None)
        if hook is not None:
            res = hook(res)
        self.futures.set_result(rid, res)

    def enqueue(self, op: str, model_id: str, payload: Dict[str, Any], seq_id: Optional[int] = None,
                post=None) -> T.UntypedAPIFuture:
        if model_id not in self.models:
            raise HTTPException(404, f"unknown model_id {model_id!r}")
        self.touch()
        rid = self.futures.create(op, model_id)
        if post is not None:
            self._post[rid] = post
        self.orch.submit(OrchestratorRequest(request_id=rid, op=op, model_id=model_id, payload=payload,
                                             seq_id=seq_id))
        return T.UntypedAPIFuture(request_id=rid, model_id=model_id)

    def touch(self) -> None:
        self.last_activity = time.time()

    def check_storage(self) -> None:
        """507 before a save when the files under the output directory already exceed the limit
        (src/xorl/server/api_server/weights.py:692-697)."""
        if self.storage_limit_bytes <= 0 or not os.path.isdir(self.output_dir):
            return
        used = 0
        for root, _dirs, files in os.walk(self.output_dir):
            for f in files:
                try:
                    used += os.path.getsize(os.path.join(root, f))
                except OSError:
                    pass
        if used >= self.storage_limit_bytes:
            raise HTTPException(507, f"storage limit reached: {used} of {self.storage_limit_bytes} bytes used under "
                                     f"the output directory; delete checkpoints first")

    # ---- sessions --------------------------------------------------------------------------
    def expire_sessions(self, now: Optional[float] = None) -> List[str]:
        now = time.time() if now is None else now
        dead = [s for s, v in self.sessions.items() if now - v["last_heartbeat"] > self.session_timeout]
        for s in dead:
            self.kill_session(s)
        return dead

    def kill_session(self, sid: str) -> List[str]:
        info = self.sessions.pop(sid, None)
        released = []
        if info:
            for mid in info["models"]:
                if mid != "default" and mid in self.models:
                    self.backend.unload_model(mid)
                    del self.models[mid]
                    released.append(mid)
        return released

    def maybe_idle_sleep(self, now: Optional[float] = None) -> bool:
        now = time.time() if now is None else now
        if self.idle_sleep_seconds > 0 and not self.asleep and self.futures.pending() == 0 \
                and now - self.last_activity > self.idle_sleep_seconds:
            self.backend.sleep()
            self.asleep = True
            return True
        return False

    def weights_dir(self, model_id: str) -> str:
        return os.path.join(self.output_dir, "weights", model_id)


def create_app(state: ServerState) -> FastAPI:
    @contextlib.asynccontextmanager
    async def lifespan(_app):
        state.orch.start()
        yield
        state.orch.stop()

    app = FastAPI(title="xorl_b200 training service", lifespan=lifespan)
    app.state.server = state

    def auth(authorization: Optional[str] = Header(default=None), x_api_key: Optional[str] = Header(default=None)):
        if not state.api_keys:
            return
        tok = x_api_key or (authorization[7:] if authorization and authorization.startswith("Bearer ") else None)
        if tok not in state.api_keys:
            raise HTTPException(401, "invalid or missing API key")

    dep = [Depends(auth)]

    # ---- health ------------------------------------------------------------------------------
    @app.get("/")
    def root():
        return {"service": "xorl_b200", "uptime": time.time() - state.started}

    @app.get("/health")
    @app.get("/api/v1/healthz")
    def health():
        return {"status": "ok", "queue_depth": state.orch.queue_depth(), "pending": state.futures.pending(),
                "asleep": state.asleep, "backend": state.backend.health()}

    # ---- training ----------------------------------------------------------------------------
    def _fb_post(n_datums):
        def post(res):
            lps = res.get("logprobs") or [[] for _ in range(n_datums)]
            outs = [{"logprobs": T.TensorData(data=lp, dtype="float32", shape=[len(lp)]).model_dump()} for lp in lps]
            metrics = dict(res.get("metrics", {}))
            if "loss" in res:
                metrics.setdefault("loss:sum", float(res["loss"]))
            return {"type": "forward_backward", "loss_fn_output_type": "logprobs", "loss_fn_outputs": outs,
                    "metrics": metrics}
        return post

    @app.post("/api/v1/forward_backward", dependencies=dep)
    def forward_backward(req: T.ForwardBackwardRequest):
        inp = req.forward_backward_input
        if not inp.data:
            raise HTTPException(422, "forward_backward_input.data is empty")
        payload = {"datums": [_datum_to_dict(d) for d in inp.data], "loss_fn": inp.loss_fn,
                   "loss_fn_config": inp.loss_fn_config}
        return state.enqueue("forward_backward", req.model_id, payload, req.seq_id, _fb_post(len(inp.data)))

    @app.post("/api/v1/forward", dependencies=dep)
    def forward(req: T.ForwardRequest):
        inp = req.forward_input
        if not inp.data:
            raise HTTPException(422, "forward_input.data is empty")
        payload = {"datums": [_datum_to_dict(d) for d in inp.data], "loss_fn": inp.loss_fn,
                   "loss_fn_config": inp.loss_fn_config}
        return state.enqueue("forward", req.model_id, payload, req.seq_id, _fb_post(len(inp.data)))

    @app.post("/api/v1/optim_step", dependencies=dep)
    def optim_step(req: T.OptimStepRequest):
        payload = {"adam_params": req.adam_params.model_dump(), "gradient_clip": req.gradient_clip}
        return state.enqueue("optim_step", req.model_id, payload, req.seq_id,
                             lambda r: {"type": "optim_step", "metrics": r.get("metrics", {})})

    @app.post("/api/v1/abort_gradient_epoch", dependencies=dep)
    def abort_epoch(req: T.AbortGradientEpochRequest):
        return state.enqueue("abort_gradient_epoch", req.model_id, {})

    @app.post("/api/v1/retrieve_future", dependencies=dep)
    def retrieve(req: T.FutureRetrieveRequest):
        e = state.futures.get(req.request_id)
        if e is None:
            raise HTTPException(404, f"unknown request_id {req.request_id}")
        if e["state"] == "pending":
            return T.TryAgainResponse(request_id=req.request_id,
                                      queue_state="paused" if state.asleep else "active")
        if e["state"] == "failed":
            return T.RequestFailedResponse(request_id=req.request_id, error=e["error"],
                                           category=e.get("category", "server"))
        return e["result"]

    # ---- models / sessions ---------------------------------------------------------------------
    @app.post("/api/v1/create_model", dependencies=dep)
    def create_model(req: T.CreateModelRequest):
        mid = req.model_id or f"model-{uuid.uuid4().hex[:8]}"
        try:
            validate_identifier(mid, "model_id")          # becomes a directory name under weights/
        except ValueError as e:
            raise HTTPException(422, str(e)) from None
        if mid in state.models and mid != "default":
            raise HTTPException(409, f"model {mid} exists")
        state.backend.create_model(mid, base_model=req.base_model, lora_config=req.lora_config)
        state.models[mid] = {"model_id": mid, "created": time.time(), "base_model": req.base_model,
                             "lora_config": req.lora_config, "session_id": req.session_id}
        if req.session_id in state.sessions:
            state.sessions[req.session_id]["models"].append(mid)
        state.training_runs[mid] = {"training_run_id": mid, "base_model": req.base_model,
                                    "is_lora": req.lora_config is not None, "created": time.time()}
        return {"model_id": mid, "is_lora": req.lora_config is not None}

    @app.post("/api/v1/unload_model", dependencies=dep)
    def unload_model(req: T.UnloadModelRequest):
        if req.model_id not in state.models:
            raise HTTPException(404, f"unknown model_id {req.model_id!r}")
        state.backend.unload_model(req.model_id)
        if req.model_id != "default":
            del state.models[req.model_id]
        return {"model_id": req.model_id, "unloaded": True}

    @app.post("/api/v1/create_session", dependencies=dep)
    def create_session(req: T.CreateSessionRequest):
        sid = uuid.uuid4().hex
        state.sessions[sid] = {"session_id": sid, "tags": req.tags, "user_metadata": req.user_metadata,
                               "created": time.time(), "last_heartbeat": time.time(), "models": []}
        return {"session_id": sid}

    @app.post("/api/v1/session_heartbeat", dependencies=dep)
    def heartbeat(req: T.SessionHeartbeatRequest):
        s = state.sessions.get(req.session_id)
        if s is None:
            raise HTTPException(404, "unknown session")
        s["last_heartbeat"] = time.time()
        state.touch()
        return {"session_id": req.session_id, "ok": True}

    @app.get("/api/v1/session_info", dependencies=dep)
    def session_info(session_id: Optional[str] = None):
        state.expire_sessions()
        if session_id is None:
            return {"sessions": list(state.sessions.values())}
        s = state.sessions.get(session_id)
        if s is None:
            raise HTTPException(404, "unknown session")
        return s

    @app.post("/api/v1/kill_session", dependencies=dep)
    def kill_session(req: T.SessionHeartbeatRequest):
        if req.session_id not in state.sessions:
            raise HTTPException(404, "unknown session")
        return {"session_id": req.session_id, "released_models": state.kill_session(req.session_id)}

    @app.get("/api/v1/training_runs", dependencies=dep)
    def training_runs():
        return {"training_runs": list(state.training_runs.values())}

    # ---- weights -----------------------------------------------------------------------------
    @app.post("/api/v1/save_weights", dependencies=dep)
    def save_weights(req: T.SaveWeightsRequest):
        state.check_storage()
        return state.enqueue("save_weights", req.model_id, {"path": req.path}, req.seq_id,
                             lambda r: {"type": "save_weights", "path": r.get("path")})

    @app.post("/api/v1/save_weights_for_sampler", dependencies=dep)
    def save_for_sampler(req: T.SaveWeightsRequest):
        name = req.path or f"sampler-{int(time.time())}"
        try:
            validate_identifier(name, "sampler weights name")
        except ValueError as e:
            raise HTTPException(422, str(e)) from None
        if os.path.exists(os.path.join(state.output_dir, "sampler_weights", name)):
            raise HTTPException(409, f"sampler weights {name!r} exist already; use another name or delete them first")
        state.check_storage()
        return state.enqueue("save_sampler_weights", req.model_id,
                             {"name": name, "quantization": state.sync_quantization},
                             req.seq_id, lambda r: {"type": "save_weights_for_sampler", "kind": r.get("kind"),
                                                    "path": f"xorl://{req.model_id}/sampler_weights/{name}"})

    @app.post("/api/v1/load_weights", dependencies=dep)
    def load_weights(req: T.LoadWeightsRequest):
        return state.enqueue("load_weights", req.model_id, {"path": req.path, "load_optimizer": req.load_optimizer},
                             None, lambda r: {"type": "load_weights", "path": r.get("path")})

    @app.get("/api/v1/list_checkpoints", dependencies=dep)
    def list_checkpoints(model_id: str = "default"):
        d = state.weights_dir(model_id)
        names = sorted(os.listdir(d)) if os.path.isdir(d) else []
        return {"checkpoints": [{"name": n, "path": f"xorl://{model_id}/weights/{n}",
                                 "mtime": os.path.getmtime(os.path.join(d, n))} for n in names]}

    @app.post("/api/v1/delete_checkpoint", dependencies=dep)
    def delete_checkpoint(req: T.DeleteCheckpointRequest):
        try:
            validate_identifier(req.name, "checkpoint name")
            validate_identifier(req.model_id, "model_id")
        except ValueError as e:
            raise HTTPException(422, str(e)) from None
        p = os.path.join(state.weights_dir(req.model_id), req.name)
        if not os.path.isdir(p):
            raise HTTPException(404, f"no checkpoint {req.name}")
        shutil.rmtree(p)
        return {"deleted": req.name}

    @app.get("/api/v1/weights_info", dependencies=dep)
    def weights_info(model_id: str = "default"):
        if model_id not in state.models:
            raise HTTPException(404, f"unknown model_id {model_id!r}")
        return {**state.models[model_id], "sync_quantization": state.sync_quantization}

    # ---- inference engines -------------------------------------------------------------------
    @app.post("/add_inference_endpoint", dependencies=dep)
    def add_endpoint(req: T.InferenceEndpoint):
        # the trainer will send HTTP requests and weight broadcasts there: refuse malformed,
        # link-local, multicast and reserved targets (and anything off the allow-list when
        # XORL_REQUIRE_ENDPOINT_ALLOWLIST=1).  Only (host, port) is stored; the same checks run again
        # on every later request, on the address that request will actually contact.
        try:
            return state.endpoints.add(req.url, req.world_size, req.name)
        except ValueError as e:
            raise HTTPException(422, str(e)) from None

    @app.post("/remove_inference_endpoint", dependencies=dep)
    def remove_endpoint(req: T.InferenceEndpoint):
        if not state.endpoints.remove(req.url):
            raise HTTPException(404, "unknown endpoint")
        return {"removed": req.url}

    @app.get("/list_inference_endpoints", dependencies=dep)
    def list_endpoints():
        return {"endpoints": state.endpoints.list()}

    @app.post("/api/v1/create_sampling_session", dependencies=dep)
    def create_sampling_session(req: T.CreateSessionRequest):
        eps = state.endpoints.list()
        if not eps:
            raise HTTPException(409, "no inference endpoint registered")
        return {"sampling_session_id": uuid.uuid4().hex, "endpoint": eps[0]["url"]}

    @app.post("/api/v1/set_sync_quantization", dependencies=dep)
    def set_sync_quant(req: T.SetSyncQuantizationRequest):
        state.sync_quantization = None if req.format in (None, "bf16") else req.format
        return {"format": state.sync_quantization or "bf16"}

    @app.post("/api/v1/sync_inference_weights", dependencies=dep)
    @app.post("/sync_inference_weights", dependencies=dep)
    def sync_weights(req: T.SyncWeightsRequest):
        payload = {"backend": req.backend, "quantization": req.quantization or state.sync_quantization,
                   "bucket_size_mb": req.bucket_size_mb}
        return state.enqueue("sync_inference_weights", req.model_id, payload, None,
                             lambda r: {"type": "sync_inference_weights", **r})

    @app.post("/sleep", dependencies=dep)
    def sleep():
        state.backend.sleep()
        state.asleep = True
        return {"asleep": True}

    @app.post("/wake_up", dependencies=dep)
    def wake_up():
        state.backend.wake_up()
        state.asleep = False
        state.touch()
        return {"asleep": False}

    return app
