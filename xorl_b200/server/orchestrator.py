"""Request queue and scheduling between the API process and the worker fleet.

Requests are executed one at a time in an order chosen by a policy: plain FIFO, or seq-id aware
FIFO — requests of one model carrying sequence ids run in increasing seq-id order even if they
arrive out of order, as the client library pipelines forward_backward / optim_step calls
(src/xorl/server/orchestrator/scheduler.py:511-979).  ``forward_backward`` payloads are packed into
micro-batches per data-parallel rank before they reach the backend
(src/xorl/server/orchestrator/request_processor.py)."""
from __future__ import annotations

import threading
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Any, Callable, Deque, Dict, List, Optional

from .packing import apply_oversized_policy, balance_across_dp, pack_balanced_dp, pack_best_fit, pack_sequential


@dataclass
class OrchestratorRequest:
    request_id: str
    op: str
    model_id: str = "default"
    seq_id: Optional[int] = None
    payload: Dict[str, Any] = field(default_factory=dict)
    created: float = field(default_factory=time.time)
    aborted: bool = False


class FIFOPolicy:
    def __init__(self):
        self.q: Deque[OrchestratorRequest] = deque()

    def push(self, r: OrchestratorRequest) -> None:
        self.q.append(r)

    def pop(self) -> Optional[OrchestratorRequest]:
        while self.q:
            r = self.q.popleft()
            if not r.aborted:
                return r
        return None

    def abort(self, request_id: str) -> bool:
        for r in self.q:
            if r.request_id == request_id:
                r.aborted = True
                return True
        return False

    def __len__(self):
        return sum(1 for r in self.q if not r.aborted)


class SeqIdAwareFIFOPolicy(FIFOPolicy):
    """Per model, a request with ``seq_id`` is released only when every smaller seq id of that
    model has been released (or after ``max_wait`` seconds, so a lost request cannot stall the
    queue).  Requests without a seq id are plain FIFO."""

    def __init__(self, max_wait: float = 30.0):
        super().__init__()
        self.next_seq: Dict[str, int] = {}
        self.max_wait = max_wait

    def pop(self) -> Optional[OrchestratorRequest]:
        now = time.time()
        for r in list(self.q):
            if r.aborted:
                self.q.remove(r)
                continue
            if r.seq_id is None:
                self.q.remove(r)
                return r
            exp = self.next_seq.get(r.model_id)
            if exp is None:
                exp = min(x.seq_id for x in self.q if x.model_id == r.model_id and x.seq_id is not None
                          and not x.aborted)
            if r.seq_id <= exp or now - r.created > self.max_wait:
                self.q.remove(r)
                self.next_seq[r.model_id] = max(exp, r.seq_id) + 1
                return r
        return None


class RequestProcessor:
    """Turns API payloads into backend calls (datum packing for forward/forward_backward)."""

    PACKERS = ("sequential", "best_fit", "balanced_dp")

    def __init__(self, dp_size: int = 1, packing_len: int = 4096, packing: str = "sequential",
                 pad_to: int = 128, on_oversized: str = "error"):
        if packing not in self.PACKERS:
            raise ValueError(f"unknown packing strategy {packing!r}; expected one of {self.PACKERS}")
        self.dp, self.packing_len, self.packing, self.pad_to = dp_size, packing_len, packing, pad_to
        self.on_oversized = on_oversized

    def admit(self, datums: List[Dict[str, Any]]):
        """Applies the oversized policy.  Returns the surviving datums and their positions in the request."""
        kept, origin = apply_oversized_policy(datums, self.packing_len, self.on_oversized)
        if not kept:
            raise ValueError("every datum of the request is longer than the packing length")
        return kept, origin

    @staticmethod
    def restore_order(result: Any, origin: List[int], n: int) -> Any:
        """Per-datum lists of a result (one entry per admitted datum) back to one entry per datum of
        the request; a skipped datum gets an empty entry."""
        if not isinstance(result, dict) or len(origin) == n:
            return result
        out = dict(result)
        for k, v in result.items():
            if isinstance(v, list) and len(v) == len(origin):
                full: List[Any] = [[] for _ in range(n)]
                for o, item in zip(origin, v):
                    full[o] = item
                out[k] = full
        out["skipped_datums"] = sorted(set(range(n)) - set(origin))
        return out

    def plan(self, datums: List[Dict[str, Any]]) -> List[List[List[int]]]:
        lengths = [len(d["tokens"]) for d in datums]
        too_long = [i for i, n in enumerate(lengths) if n > self.packing_len]
        if too_long:
            raise ValueError(f"datum {too_long[0]} has {lengths[too_long[0]]} tokens, more than the "
                             f"packing length {self.packing_len}")
        if self.packing == "balanced_dp":
            bins = pack_balanced_dp(lengths, self.packing_len, self.dp)
        elif self.packing == "best_fit":
            bins = pack_best_fit(lengths, self.packing_len)
        else:
            bins = pack_sequential(lengths, self.packing_len)
        return balance_across_dp(bins, lengths, self.dp)


class Orchestrator:
    def __init__(self, backend, policy: Optional[FIFOPolicy] = None,
                 processor: Optional[RequestProcessor] = None,
                 on_result: Optional[Callable[[str, Any, Optional[str]], None]] = None):
        self.backend = backend
        self.policy = policy or SeqIdAwareFIFOPolicy()
        self.processor = processor or RequestProcessor()
        self.on_result = on_result or (lambda rid, res, err: None)
        self._cv = threading.Condition()
        self._stop = False
        self._thread: Optional[threading.Thread] = None
        self.processed = 0

    def submit(self, req: OrchestratorRequest) -> None:
        with self._cv:
            self.policy.push(req)
            self._cv.notify()

    def abort(self, request_id: str) -> bool:
        with self._cv:
            return self.policy.abort(request_id)

    def start(self) -> None:
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def stop(self) -> None:
        with self._cv:
            self._stop = True
            self._cv.notify()
        if self._thread is not None:
            self._thread.join(timeout=5)

    def queue_depth(self) -> int:
        with self._cv:
            return len(self.policy)

    def _loop(self) -> None:
        while True:
            with self._cv:
                req = self.policy.pop()
                while req is None and not self._stop:
                    self._cv.wait(timeout=0.05)
                    req = self.policy.pop()
                if req is None and self._stop:
                    return
            self._execute(req)

    def _execute(self, req: OrchestratorRequest) -> None:
        try:
            if req.op in ("forward_backward", "forward"):
                requested = req.payload["datums"]
                datums, origin = self.processor.admit(requested)
                plan = self.processor.plan(datums)
                res = getattr(self.backend, req.op)(req.model_id, datums, plan, req.payload.get("loss_fn", "cross_entropy"),
                                                    req.payload.get("loss_fn_config", {}))
                res = self.processor.restore_order(res, origin, len(requested))
            else:
                res = getattr(self.backend, req.op)(req.model_id, **req.payload)
            self.processed += 1
            self.on_result(req.request_id, res, None)
        except Exception as e:  # noqa: BLE001
            self.on_result(req.request_id, None, f"{type(e).__name__}: {e}")
