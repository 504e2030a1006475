"""Large request payloads that travel beside the control messages.

Rollout routing replay sends ``[tokens, moe_layers, k]`` expert indices per datum, far too much
for the JSON control path, so the API process parks such tensors in a store and passes a small
reference (``{"store": "fs", "key": ..., "sha256": ..., "nbytes": ...}``) through the orchestrator to
the runner ranks, which read them directly (src/xorl/server/side_payloads.py).  The store here is a
shared-filesystem directory (one box, or a mounted volume); the reference's RDMA transfer-engine
store is not built.  Writes are atomic (temporary file + rename), reads verify length and digest,
and entries older than the time-to-live are swept.
"""
from __future__ import annotations

import hashlib
import io
import os
import time
import uuid
from typing import Any, Dict, Optional

import torch

from .security import confine_path, validate_identifier


class PayloadError(RuntimeError):
    pass


class FilesystemPayloadStore:
    kind = "fs"

    def __init__(self, root: str, ttl_seconds: float = 3600.0, max_bytes: int = 8 << 30):
        self.root = os.path.abspath(root)
        self.ttl = float(ttl_seconds)
        self.max_bytes = int(max_bytes)
        os.makedirs(self.root, exist_ok=True)

    def _path(self, key: str):
        return confine_path(self.root, validate_identifier(key, "payload key") + ".pt")

    def put(self, obj: Any, key: Optional[str] = None) -> Dict[str, Any]:
        """Stores a tensor (or a nest of tensors / plain values) and returns its reference."""
        key = key or uuid.uuid4().hex
        buf = io.BytesIO()
        torch.save(obj, buf)
        data = buf.getvalue()
        if len(data) > self.max_bytes:
            raise PayloadError(f"payload of {len(data)} bytes exceeds the limit of {self.max_bytes}")
        path = self._path(key)
        tmp = f"{path}.{uuid.uuid4().hex}.tmp"
        with open(tmp, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
        os.replace(tmp, path)
        return {"store": self.kind, "key": key, "nbytes": len(data), "sha256": hashlib.sha256(data).hexdigest()}

    def get(self, ref: Dict[str, Any], delete: bool = False) -> Any:
        if ref.get("store") != self.kind:
            raise PayloadError(f"reference belongs to store {ref.get('store')!r}, not {self.kind!r}")
        path = self._path(ref["key"])
        try:
            with open(path, "rb") as f:
                data = f.read()
        except FileNotFoundError:
            raise PayloadError(f"payload {ref['key']} is gone (expired or never written)") from None
        if len(data) != int(ref["nbytes"]) or hashlib.sha256(data).hexdigest() != ref["sha256"]:
            raise PayloadError(f"payload {ref['key']} does not match its reference (length or digest)")
        if delete:
            self.delete(ref)
        return torch.load(io.BytesIO(data), map_location="cpu", weights_only=True)

    def delete(self, ref: Dict[str, Any]) -> bool:
        try:
            os.unlink(self._path(ref["key"]))
            return True
        except FileNotFoundError:
            return False

    def sweep(self, now: Optional[float] = None) -> int:
        """Removes entries (and abandoned temporary files) older than the time-to-live."""
        now = time.time() if now is None else now
        removed = 0
        for name in os.listdir(self.root):
            p = os.path.join(self.root, name)
            try:
                if now - os.path.getmtime(p) > self.ttl:
                    os.unlink(p)
                    removed += 1
            except FileNotFoundError:
                pass
        return removed


def is_payload_ref(x: Any) -> bool:
    return isinstance(x, dict) and {"store", "key", "nbytes", "sha256"} <= set(x)


def resolve_refs(obj: Any, store: FilesystemPayloadStore) -> Any:
    """Replaces every payload reference inside a nest of dicts / lists by its content."""
    if is_payload_ref(obj):
        return store.get(obj)
    if isinstance(obj, dict):
        return {k: resolve_refs(v, store) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(resolve_refs(v, store) for v in obj)
    return obj
