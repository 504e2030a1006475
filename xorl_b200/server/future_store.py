"""Two-phase future store: a request id is handed out immediately, the result is filled in when
the orchestrator reports back, clients poll.  Entries expire after a TTL
(src/xorl/server/api_server/future_store.py:464-511)."""
from __future__ import annotations

import threading
import time
import uuid
from typing import Any, Dict, Optional


class FutureStore:
    def __init__(self, ttl_seconds: float = 3600.0):
        self.ttl = ttl_seconds
        self._lock = threading.Lock()
        self._entries: Dict[str, Dict[str, Any]] = {}

    def create(self, kind: str, model_id: Optional[str] = None) -> str:
        rid = uuid.uuid4().hex
        with self._lock:
            self._entries[rid] = {"kind": kind, "model_id": model_id, "state": "pending",
                                  "created": time.time(), "result": None, "error": None}
        return rid

    def set_result(self, rid: str, result: Any) -> None:
        with self._lock:
            e = self._entries.get(rid)
            if e is not None and e["state"] == "pending":
                e.update(state="done", result=result, finished=time.time())

    def set_error(self, rid: str, error: str, category: str = "server") -> None:
        with self._lock:
            e = self._entries.get(rid)
            if e is not None and e["state"] == "pending":
                e.update(state="failed", error=error, category=category, finished=time.time())

    def abort(self, rid: str) -> bool:
        with self._lock:
            e = self._entries.get(rid)
            if e is not None and e["state"] == "pending":
                e.update(state="failed", error="aborted", category="aborted", finished=time.time())
                return True
        return False

    def get(self, rid: str) -> Optional[Dict[str, Any]]:
        with self._lock:
            e = self._entries.get(rid)
            return dict(e) if e is not None else None

    def pending(self) -> int:
        with self._lock:
            return sum(1 for e in self._entries.values() if e["state"] == "pending")

    def cleanup(self, now: Optional[float] = None) -> int:
        now = time.time() if now is None else now
        with self._lock:
            dead = [k for k, e in self._entries.items()
                    if now - e.get("finished", e["created"]) > self.ttl]
            for k in dead:
                del self._entries[k]
        return len(dead)
