"""Backends the orchestrator drives: an abstract interface, a dummy with delay / failure injection
for service-plane tests, and a local in-process backend around a ``ModelRunner``
(src/xorl/server/backend/{base,dummy,remote}.py)."""
from __future__ import annotations

import random
import time
from typing import Any, Dict, List, Optional


class Backend:
    def forward_backward(self, model_id, datums, plan, loss_fn, loss_fn_config) -> Dict[str, Any]:
        raise NotImplementedError

    def forward(self, model_id, datums, plan, loss_fn, loss_fn_config) -> Dict[str, Any]:
        raise NotImplementedError

    def optim_step(self, model_id, **kw) -> Dict[str, Any]:
        raise NotImplementedError

    def save_weights(self, model_id, **kw) -> Dict[str, Any]:
        raise NotImplementedError

    def load_weights(self, model_id, **kw) -> Dict[str, Any]:
        raise NotImplementedError

    def sync_inference_weights(self, model_id, **kw) -> Dict[str, Any]:
        raise NotImplementedError

    def save_sampler_weights(self, model_id, **kw) -> Dict[str, Any]:
        raise NotImplementedError

    def abort_gradient_epoch(self, model_id, **kw) -> Dict[str, Any]:
        raise NotImplementedError

    def create_model(self, model_id, **kw) -> Dict[str, Any]:
        return {"model_id": model_id}

    def unload_model(self, model_id, **kw) -> Dict[str, Any]:
        return {"model_id": model_id}

    def sleep(self, model_id="default", **kw) -> Dict[str, Any]:
        return {}

    def wake_up(self, model_id="default", **kw) -> Dict[str, Any]:
        return {}

    def health(self) -> Dict[str, Any]:
        return {"status": "ok"}


class DummyBackend(Backend):
    """Answers every call after ``processing_delay`` seconds; fails with probability
    ``failure_rate`` (fault injection for the API / orchestrator tests)."""

    def __init__(self, processing_delay: float = 0.0, failure_rate: float = 0.0, seed: int = 0):
        self.delay, self.failure_rate = processing_delay, failure_rate
        self.rng = random.Random(seed)
        self.calls: List[str] = []
        self.steps = 0

    def _maybe_fail(self, op: str) -> None:
        self.calls.append(op)
        if self.delay:
            time.sleep(self.delay)
        if self.rng.random() < self.failure_rate:
            raise RuntimeError(f"injected failure in {op}")

    def forward_backward(self, model_id, datums, plan, loss_fn, loss_fn_config):
        self._maybe_fail("forward_backward")
        n = sum(len(d["tokens"]) for d in datums)
        return {"loss": 1.0, "num_tokens": n, "logprobs": [[-1.0] * len(d["tokens"]) for d in datums],
                "metrics": {"loss:sum": float(n)}}

    def forward(self, model_id, datums, plan, loss_fn, loss_fn_config):
        self._maybe_fail("forward")
        return {"logprobs": [[-1.0] * len(d["tokens"]) for d in datums], "metrics": {}}

    def optim_step(self, model_id, **kw):
        self._maybe_fail("optim_step")
        self.steps += 1
        return {"metrics": {"grad_norm": 1.0, "step": float(self.steps)}}

    def save_weights(self, model_id, **kw):
        self._maybe_fail("save_weights")
        return {"path": kw.get("path") or f"xorl://{model_id}/weights/dummy"}

    def load_weights(self, model_id, **kw):
        self._maybe_fail("load_weights")
        return {"path": kw.get("path")}

    def sync_inference_weights(self, model_id, **kw):
        self._maybe_fail("sync_inference_weights")
        return {"synced": True, "bytes": 0}

    def save_sampler_weights(self, model_id, **kw):
        self._maybe_fail("save_sampler_weights")
        return {"kind": "full_weights", "directory": kw.get("name")}

    def abort_gradient_epoch(self, model_id, **kw):
        self.calls.append("abort_gradient_epoch")
        return {"aborted": True}


class LocalBackend(Backend):
    """Runs a ``ModelRunner`` in this process (single-rank serving, tests)."""

    def __init__(self, runner):
        self.runner = runner

    def forward_backward(self, model_id, datums, plan, loss_fn, loss_fn_config):
        return self.runner.forward_backward(model_id, datums, plan, loss_fn, loss_fn_config)

    def forward(self, model_id, datums, plan, loss_fn, loss_fn_config):
        return self.runner.forward(model_id, datums, plan, loss_fn, loss_fn_config)

    def optim_step(self, model_id, **kw):
        return self.runner.optim_step(model_id, **kw)

    def save_weights(self, model_id, **kw):
        return self.runner.save_weights(model_id, **kw)

    def load_weights(self, model_id, **kw):
        return self.runner.load_weights(model_id, **kw)

    def sync_inference_weights(self, model_id, **kw):
        return self.runner.sync_inference_weights(model_id, **kw)

    def save_sampler_weights(self, model_id, **kw):
        return self.runner.save_sampler_weights(model_id, **kw)

    def abort_gradient_epoch(self, model_id, **kw):
        return self.runner.abort_gradient_epoch(model_id)

    def create_model(self, model_id, **kw):
        return self.runner.create_model(model_id, **kw)

    def unload_model(self, model_id, **kw):
        return self.runner.unload_model(model_id, **kw)

    def sleep(self, model_id="default", **kw):
        return self.runner.sleep()

    def wake_up(self, model_id="default", **kw):
        return self.runner.wake_up()
