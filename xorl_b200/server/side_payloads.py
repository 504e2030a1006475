"""Large request payloads that travel beside the control messages.

Rollout routing replay sends ``[tokens, moe_layers, k]`` expert indices per datum, far too much
for the JSON control path, so the API process parks such tensors in a store and passes a small
reference (``{"store": "fs", "key": ..., "sha256": ..., "nbytes": ...}``) through the orchestrator to
the runner ranks, which read them directly (src/xorl/server/side_payloads.py).  The store here is a
shared-filesystem directory (one box, or a mounted volume); the reference's RDMA transfer-engine
store is not built.  Writes are atomic (temporary file + rename), reads verify length and digest,
and entries older than the time-to-live are swept.

``RoutingPayloads`` is the routing-replay use of it: before rank 0 broadcasts a command to the fleet, the
``routed_experts`` of all datums are packed row after row into a few large chunk files (int16 expert ids,
-1 = keep the router's choice) and each datum keeps a reference to its rows; a rank reads only the rows of
the datums it runs (a seek and a read, checked against the datum's checksum), and the chunks are removed
when the command has run on every rank -- also when it failed.
"""
from __future__ import annotations

import hashlib
import io
import os
import time
import uuid
import zlib
from typing import Any, Dict, List, Optional, Tuple

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


# ---------------------------------------------------------------------------------------------
# routing replay payloads
# ---------------------------------------------------------------------------------------------
ROUTING_KIND = "r3_routing"
ROUTING_FIELD = "routed_experts"


def is_routing_ref(x: Any) -> bool:
    return isinstance(x, dict) and x.get("kind") == ROUTING_KIND and "chunk" in x


def canonical_routing(item: Any) -> torch.Tensor:
    """``[tokens, moe_layers, k]`` int16 from nested lists, a tensor, or the inference engine's encoded form
    ``{"data": base64 of little-endian integers, "shape": [...], "dtype": "int16" | "int32" | "uint8"}``."""
    if isinstance(item, dict) and "data" in item and "shape" in item:
        import base64
        import numpy as np
        raw = base64.b64decode(item["data"])
        arr = np.frombuffer(raw, dtype=np.dtype(item.get("dtype", "int32")).newbyteorder("<")).reshape(item["shape"])
        t = torch.from_numpy(arr.astype("int64"))
    else:
        t = torch.as_tensor(item)
    if t.dim() != 3:
        raise PayloadError(f"routed_experts must be [tokens, moe_layers, k], got shape {tuple(t.shape)}")
    if t.numel() and (int(t.max()) > 32767 or int(t.min()) < -1):
        raise PayloadError("routed_experts holds an expert id outside -1..32767")
    return t.to(torch.int16).contiguous()


class RoutingPayloads:
    def __init__(self, store: FilesystemPayloadStore, chunk_bytes: int = 256 << 20, min_bytes: int = 1 << 16):
        self.store = store
        self.chunk_bytes = int(chunk_bytes)
        self.min_bytes = int(min_bytes)              # smaller requests stay inline in the command

    def _chunk_path(self, key: str) -> str:
        return str(confine_path(self.store.root, validate_identifier(key, "payload key") + ".rows"))

    def stash(self, datums: List[Dict[str, Any]]) -> Tuple[List[Dict[str, Any]], List[str]]:
        """(datums with ``routed_experts`` replaced by references, chunk keys to clean up).  Datums without
        routing, and requests whose routing is small, pass through untouched."""
        tensors = {i: canonical_routing(d[ROUTING_FIELD]) for i, d in enumerate(datums)
                   if d.get(ROUTING_FIELD) is not None and not is_routing_ref(d[ROUTING_FIELD])}
        if sum(t.numel() * 2 for t in tensors.values()) < self.min_bytes:
            return datums, []
        out = [dict(d) for d in datums]
        keys: List[str] = []
        cur: List[Tuple[int, torch.Tensor]] = []
        size = 0

        def flush():
            nonlocal cur, size
            if not cur:
                return
            key = uuid.uuid4().hex
            path = self._chunk_path(key)
            tmp = f"{path}.{uuid.uuid4().hex}.tmp"
            offset = 0
            try:
                with open(tmp, "wb") as f:
                    for i, t in cur:
                        data = t.numpy().tobytes()
                        f.write(data)
                        out[i][ROUTING_FIELD] = {"kind": ROUTING_KIND, "store": self.store.kind, "chunk": key,
                                                 "offset": offset, "nbytes": len(data), "shape": list(t.shape),
                                                 "dtype": "int16", "crc32": zlib.crc32(data)}
                        offset += len(data)
                    f.flush()
                    os.fsync(f.fileno())
                os.replace(tmp, path)
            except BaseException:
                # nothing half-written stays behind, and what this call already stored goes too
                for p in (tmp, path):
                    try:
                        os.unlink(p)
                    except FileNotFoundError:
                        pass
                self.cleanup(keys)
                raise
            keys.append(key)
            cur, size = [], 0

        for i, t in tensors.items():
            nb = t.numel() * 2
            if cur and size + nb > self.chunk_bytes:
                flush()
            cur.append((i, t))
            size += nb
        flush()
        return out, keys

    def load(self, ref: Dict[str, Any]) -> torch.Tensor:
        """The rows of one datum, ``[tokens, moe_layers, k]`` int64."""
        import numpy as np
        if not is_routing_ref(ref) or ref.get("store") != self.store.kind:
            raise PayloadError("not a routing payload reference of this store")
        try:
            with open(self._chunk_path(ref["chunk"]), "rb") as f:
                f.seek(int(ref["offset"]))
                data = f.read(int(ref["nbytes"]))
        except FileNotFoundError:
            raise PayloadError(f"routing payload chunk {ref['chunk']} is gone (expired or cleaned up)") from None
        if len(data) != int(ref["nbytes"]) or zlib.crc32(data) != int(ref["crc32"]):
            raise PayloadError(f"routing payload rows of chunk {ref['chunk']} do not match their reference")
        return torch.from_numpy(np.frombuffer(data, dtype="<i2").reshape(ref["shape"]).astype("int64"))

    def resolve(self, datum: Dict[str, Any]) -> Dict[str, Any]:
        r = datum.get(ROUTING_FIELD)
        if is_routing_ref(r):
            datum = dict(datum)
            datum[ROUTING_FIELD] = self.load(r)
        return datum

    def cleanup(self, keys: List[str]) -> Dict[str, int]:
        deleted = freed = 0
        for k in keys:
            p = self._chunk_path(k)
            try:
                freed += os.path.getsize(p)
                os.unlink(p)
                deleted += 1
            except FileNotFoundError:
                pass
        return {"chunks_deleted": deleted, "bytes_freed": freed}
