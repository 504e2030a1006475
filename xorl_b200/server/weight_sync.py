"""Pushing trained weights to inference engines.

* ``EndpointManager`` keeps the registered engines and talks to their control routes
  (``/health``, ``/pause_generation``, ``/init_weights_update_group``,
  ``/update_weights_from_distributed``, ``/continue_generation``), cf.
  src/xorl/server/weight_sync/endpoint_manager.py.
* ``iter_sync_tensors`` walks the sharded model unit by unit, gathers each unit once, splits fused
  projections back into the names an inference engine knows, optionally quantises (block fp8 with
  ``_scale_inv`` companions), and groups tensors into buckets of a bounded size.
* Transports: ``StatelessGroupBroadcaster`` (a process group of 1 + sum(engine world) ranks built
  directly on a TCP store, bucketed broadcast from rank 0 -- src/xorl/server/weight_sync/backends/
  nccl_broadcast.py:326-390), ``PeerCopyTransport`` (one copy kernel per bucket straight into the
  engine's device buffers mapped through CUDA IPC on the same box), ``FileTransport`` (safetensors
  buckets in a shared directory) and ``SparseDeltaTransport`` (only the 16-bit words that changed
  since the previous sync, C++ codec -- src/xorl/server/weight_sync/backends/sparse_delta.py:205).
"""
from __future__ import annotations

import ctypes
import json
import os
import time
from datetime import timedelta
from typing import Any, Callable, Dict, Iterator, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..checkpoint.handlers import get_checkpoint_handler
from ..ops import _lib
from ..ops import quantize as Q


# ---------------------------------------------------------------------------------------------
# endpoints
# ---------------------------------------------------------------------------------------------
def split_endpoint(url: str) -> Tuple[str, int]:
    """``http://host:port`` (scheme optional) -> (host, port).  Inference endpoints are plain HTTP
    inside the cluster; anything else is refused."""
    from urllib.parse import urlsplit
    u = urlsplit(url if "//" in url else "http://" + url)
    if u.scheme != "http" or not u.hostname:
        raise ValueError(f"endpoint URL {url!r} needs an http host")
    if u.path not in ("", "/") or u.query or u.fragment or u.username or u.password:
        raise ValueError(f"endpoint URL {url!r} must be just http://host:port")
    try:
        port = u.port or 80
    except ValueError:
        raise ValueError(f"endpoint URL {url!r} has an invalid port") from None
    return u.hostname, port


class EndpointManager:
    """Registered inference engines.  An endpoint is kept as ``(host, port)``; every outbound request
    URL is rebuilt at the moment of use by ``url_of`` (default ``security.endpoint_url``), which
    resolves the host again, re-applies the address checks and returns an address literal, so a
    hostname whose DNS answer changes after registration cannot move the request to an unsafe
    address (src/xorl/server/weight_sync/backends/nccl_broadcast.py:536-867 builds its URLs the
    same way)."""

    def __init__(self, post: Optional[Callable[[str, Dict[str, Any]], Dict[str, Any]]] = None,
                 get: Optional[Callable[[str], Dict[str, Any]]] = None, timeout: float = 300.0,
                 url_of: Optional[Callable[[str, int, str], str]] = None):
        self.endpoints: Dict[str, Dict[str, Any]] = {}
        self.timeout = timeout
        self._post = post or self._http_post
        self._get = get or self._http_get
        self._url_of = url_of or self._checked_url

    @staticmethod
    def _checked_url(host: str, port: int, path: str) -> str:
        from .security import endpoint_url
        return endpoint_url(host, port, path,
                            require_allowlist=os.environ.get("XORL_REQUIRE_ENDPOINT_ALLOWLIST", "0") == "1")

    def _http_post(self, url, payload):
        import requests
        r = requests.post(url, json=payload, timeout=self.timeout, allow_redirects=False)
        r.raise_for_status()
        return r.json() if r.content else {}

    def _http_get(self, url):
        import requests
        r = requests.get(url, timeout=self.timeout, allow_redirects=False)
        r.raise_for_status()
        return r.json() if r.content else {}

    @staticmethod
    def _key(url: str) -> str:
        host, port = split_endpoint(url)
        return f"http://[{host}]:{port}" if ":" in host else f"http://{host}:{port}"

    def add(self, url: str, world_size: int = 1, name: Optional[str] = None) -> Dict[str, Any]:
        host, port = split_endpoint(url)
        self._url_of(host, port, "/health")          # refuses unsafe targets at registration too
        key = self._key(url)
        info = {"url": key, "host": host, "port": port, "world_size": int(world_size),
                "name": name or key, "added": time.time(), "healthy": None}
        self.endpoints[key] = info
        return info

    def remove(self, url: str) -> bool:
        try:
            return self.endpoints.pop(self._key(url), None) is not None
        except ValueError:
            return False

    def list(self) -> List[Dict[str, Any]]:
        return list(self.endpoints.values())

    def total_world(self) -> int:
        return sum(e["world_size"] for e in self.endpoints.values())

    def request_url(self, endpoint: Dict[str, Any], path: str) -> str:
        """The URL to contact for ``path`` right now (validated address literal)."""
        return self._url_of(endpoint["host"], endpoint["port"], path)

    def check_health(self) -> Dict[str, bool]:
        out = {}
        for key, e in self.endpoints.items():
            try:
                self._get(self.request_url(e, "/health"))
                e["healthy"] = True
            except Exception:  # noqa: BLE001
                e["healthy"] = False
            out[key] = e["healthy"]
        return out

    def broadcast_post(self, route: str, payload_of: Callable[[Dict[str, Any], int], Dict[str, Any]]):
        """POST to every endpoint; ``payload_of(endpoint, rank_offset)`` builds the body, where
        ``rank_offset`` is the first sync-group rank of that endpoint (rank 0 is the trainer)."""
        out, offset = [], 1
        for e in self.endpoints.values():
            out.append(self._post(self.request_url(e, route), payload_of(e, offset)))
            offset += e["world_size"]
        return out


# ---------------------------------------------------------------------------------------------
# tensor stream
# ---------------------------------------------------------------------------------------------
def _quantise(name: str, t: torch.Tensor, fmt: Optional[str], selected: Optional[bool] = None
              ) -> List[Tuple[str, torch.Tensor]]:
    """``selected``: None = every 2-D projection weight is converted (by name); True / False = the caller
    knows whether this weight's module is one of the modules to convert (a fake-quantised model exports
    exactly the weights it trained on the grid)."""
    if fmt in (None, "bf16") or t.dim() != 2 or not name.endswith(".weight") or selected is False:
        return [(name, t)]
    if selected is None and ("embed" in name or "lm_head" in name or "norm" in name or ".gate.weight" in name):
        return [(name, t)]
    if fmt == "fp8":
        if t.shape[0] % 128 or t.shape[1] % 128:
            return [(name, t)]
        q, s = Q.block_fp8_quantize_128x128(t.float())
        return [(name, q.view(torch.uint8)), (name + "_scale_inv", s)]
    if fmt == "nvfp4":
        packed, bs, gs = Q.nvfp4_quantize(t.float())
        return [(name, packed), (name + "_scale", bs), (name + "_scale_2", gs.reshape(1))]
    raise ValueError(f"unknown sync quantization {fmt!r}")


def iter_sync_tensors(engine, cfg, dtype=torch.bfloat16, quantization: Optional[str] = None,
                      merged_lora: Optional[Callable[[str, torch.Tensor], torch.Tensor]] = None,
                      only_modules: Optional[set] = None) -> Iterator[Tuple[str, torch.Tensor]]:
    """(engine-side name, tensor) for every weight, in model order.  All ranks of the shard groups
    must iterate together (the gathers are collectives); only the consumer on rank 0 uses them."""
    handler = get_checkpoint_handler(cfg)

    def local():
        for fqn, full in engine.iter_full_tensors("master"):
            if ".lora_" in fqn or "_lora_" in fqn or ".lora." in fqn:
                continue
            t = full
            if merged_lora is not None:
                t = merged_lora(fqn, t)
            t = t.to(dtype)
            sel = None if only_modules is None else fqn.rsplit(".", 1)[0] in only_modules
            for name, part in handler.to_hf(fqn, t):
                yield from _quantise(name, part, quantization, sel)

    ps = engine.ps
    if getattr(ps, "pp_size", 1) <= 1 or not dist.is_initialized():
        yield from local()
        return
    yield from _relay_pipeline_stages(local(), ps, engine.device)


def _relay_pipeline_stages(stream, ps, device) -> Iterator[Tuple[str, torch.Tensor]]:
    """Under pipeline parallelism every stage holds its own layers.  The ranks that share global rank
    0's data / tensor coordinates (one per stage: rank 0's pipeline group) forward their stage's tensors
    to rank 0 one by one, in stage order, so the driver sees the whole model in model order
    (src/xorl/server/weight_sync/handler.py ``_extract_params_for_sync`` with the PP transfer path).
    Every rank drains its own stage's stream (the gathers inside are collective over the stage)."""
    mine = ps.group_ranks("pp")
    leader = 0 in mine
    rank = ps.rank
    if not leader:
        for _ in stream:
            pass
        return
    if rank == 0:
        yield from stream
        for src in mine[1:]:
            while True:
                box = [None]
                dist.recv_object_list(box, src=src)
                if box[0] is None:
                    break
                name, shape, dt = box[0]
                t = torch.empty(shape, dtype=getattr(torch, dt), device=device)
                dist.recv(t, src=src)
                yield name, t
        return
    # a later stage's leader: wait for its turn implicitly (rank 0 receives in stage order; sends block)
    for name, t in stream:
        dist.send_object_list([(name, tuple(t.shape), str(t.dtype).replace("torch.", ""))], dst=0)
        dist.send(t.contiguous(), dst=0)
    dist.send_object_list([None], dst=0)


def bucketize(stream: Iterator[Tuple[str, torch.Tensor]], bucket_bytes: int
              ) -> Iterator[List[Tuple[str, torch.Tensor]]]:
    bucket, size = [], 0
    for name, t in stream:
        nb = t.numel() * t.element_size()
        if bucket and size + nb > bucket_bytes:
            yield bucket
            bucket, size = [], 0
        bucket.append((name, t))
        size += nb
    if bucket:
        yield bucket


def flatten_bucket(bucket: List[Tuple[str, torch.Tensor]]) -> Tuple[torch.Tensor, List[Dict[str, Any]]]:
    """One uint8 buffer (256-byte aligned entries) plus the manifest the receiver needs."""
    manifest, off = [], 0
    for name, t in bucket:
        nb = t.numel() * t.element_size()
        manifest.append({"name": name, "dtype": str(t.dtype).replace("torch.", ""), "shape": list(t.shape),
                         "offset": off, "nbytes": nb})
        off = (off + nb + 255) // 256 * 256
    flat = torch.zeros(off, dtype=torch.uint8, device=bucket[0][1].device)
    for (name, t), m in zip(bucket, manifest):
        flat[m["offset"]:m["offset"] + m["nbytes"]].copy_(t.contiguous().view(-1).view(torch.uint8))
    return flat, manifest


def unflatten_bucket(flat: torch.Tensor, manifest: List[Dict[str, Any]]) -> Dict[str, torch.Tensor]:
    out = {}
    for m in manifest:
        dt = getattr(torch, m["dtype"])
        out[m["name"]] = flat[m["offset"]:m["offset"] + m["nbytes"]].view(dt).view(m["shape"])
    return out


# ---------------------------------------------------------------------------------------------
# transports
# ---------------------------------------------------------------------------------------------
class StatelessGroupBroadcaster:
    """A process group that exists beside the default one: built on its own TCP store, so the
    trainer (rank 0) and the engines' workers (ranks 1..) need not share a launcher."""

    def __init__(self, host: str, port: int, rank: int, world: int, backend: str = "nccl",
                 device: Optional[torch.device] = None, timeout_s: float = 300.0):
        store = dist.TCPStore(host, port, world, is_master=(rank == 0),
                              timeout=timedelta(seconds=timeout_s), wait_for_workers=False)
        self.rank, self.world, self.backend = rank, world, backend
        if backend == "nccl":
            torch.cuda.set_device(device)
            opts = dist.ProcessGroupNCCL.Options()
            self.pg = dist.ProcessGroupNCCL(dist.PrefixStore("wsync", store), rank, world, opts)
        else:
            self.pg = dist.ProcessGroupGloo(dist.PrefixStore("wsync", store), rank, world,
                                            timedelta(seconds=timeout_s))
        self.store = store

    def broadcast(self, t: torch.Tensor, src: int = 0) -> None:
        opts = dist.BroadcastOptions()
        opts.rootRank = src
        opts.rootTensor = 0
        self.pg.broadcast([t], opts).wait()

    def send_bucket(self, bucket) -> List[Dict[str, Any]]:
        flat, manifest = flatten_bucket(bucket)
        self.broadcast(flat)
        return manifest

    def recv_bucket(self, manifest, device) -> Dict[str, torch.Tensor]:
        total = max(m["offset"] + m["nbytes"] for m in manifest)
        total = (total + 255) // 256 * 256
        flat = torch.empty(total, dtype=torch.uint8, device=device)
        self.broadcast(flat)
        return unflatten_bucket(flat, manifest)


class PeerCopyTransport:
    """Same-box sync: the engine exposes device buffers (one per bucket slot) whose addresses the
    trainer has mapped (CUDA IPC or symmetric memory); each bucket is written there by one copy
    kernel on the trainer's stream, without NCCL and without a staging hop."""

    def __init__(self, dst_ptr: int, dst_bytes: int, num_ctas: int = 64):
        self.dst_ptr, self.dst_bytes, self.num_ctas = int(dst_ptr), int(dst_bytes), num_ctas

    def send_bucket(self, bucket) -> List[Dict[str, Any]]:
        flat, manifest = flatten_bucket(bucket)
        if flat.numel() > self.dst_bytes:
            raise ValueError(f"bucket of {flat.numel()} bytes exceeds the mapped buffer ({self.dst_bytes})")
        if flat.is_cuda:
            nbytes = (flat.numel() + 15) // 16 * 16
            _lib.check(_lib.cuda_lib().xb_peer_copy(ctypes.c_void_p(self.dst_ptr), flat.data_ptr(), nbytes,
                                                    self.num_ctas, _lib.stream_ptr()), "xb_peer_copy")
        else:
            ctypes.memmove(self.dst_ptr, flat.data_ptr(), flat.numel())
        return manifest


class FileTransport:
    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)
        self.index: Dict[str, str] = {}
        self.n = 0

    def send_bucket(self, bucket) -> List[Dict[str, Any]]:
        from safetensors.torch import save_file
        fname = f"bucket-{self.n:05d}.safetensors"
        self.n += 1
        save_file({n: t.detach().cpu().contiguous() for n, t in bucket}, os.path.join(self.dir, fname))
        for n, _ in bucket:
            self.index[n] = fname
        return [{"name": n, "file": fname} for n, _ in bucket]

    def finish(self) -> str:
        p = os.path.join(self.dir, "model.safetensors.index.json")
        with open(p, "w") as f:
            json.dump({"metadata": {"format": "pt"}, "weight_map": self.index}, f)
        return p


def delta_encode(prev: torch.Tensor, cur: torch.Tensor) -> bytes:
    """Encodes the 16-bit words of ``cur`` that differ from ``prev`` (both CPU, same shape/dtype)."""
    lib = _lib.host_lib()
    lib.xb_delta_bound.restype = ctypes.c_longlong
    lib.xb_delta_encode.restype = ctypes.c_longlong
    a = prev.contiguous().view(torch.int16).reshape(-1)
    b = cur.contiguous().view(torch.int16).reshape(-1)
    n = a.numel()
    cap = int(lib.xb_delta_bound(ctypes.c_longlong(n)))
    out = (ctypes.c_uint8 * cap)()
    ln = lib.xb_delta_encode(ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()),
                             ctypes.c_longlong(n), out, ctypes.c_longlong(cap))
    if ln < 0:
        raise RuntimeError("delta encode failed")
    return bytes(memoryview(out)[:ln])


def delta_apply(weights: torch.Tensor, blob: bytes) -> int:
    lib = _lib.host_lib()
    lib.xb_delta_apply.restype = ctypes.c_longlong
    w = weights.view(torch.int16).reshape(-1)
    assert w.is_contiguous() and not w.is_cuda
    buf = (ctypes.c_uint8 * len(blob)).from_buffer_copy(blob)
    n = lib.xb_delta_apply(ctypes.c_void_p(w.data_ptr()), ctypes.c_longlong(w.numel()), buf,
                           ctypes.c_longlong(len(blob)))
    if n < 0:
        raise ValueError("malformed delta")
    return int(n)


class SparseDeltaTransport:
    """Writes one ``.delta`` blob per tensor that changed since the previous sync (first sync: full
    safetensors through ``FileTransport``).  Keeps the previously synced 16-bit weights on the host."""

    def __init__(self, directory: str):
        self.dir = directory
        os.makedirs(directory, exist_ok=True)
        self.prev: Dict[str, torch.Tensor] = {}
        self.generation = 0
        self.stats = {"tensors": 0, "changed_words": 0, "bytes": 0, "dense_bytes": 0}

    def begin(self) -> None:
        self.generation += 1
        self.gen_dir = os.path.join(self.dir, f"gen-{self.generation:06d}")
        os.makedirs(self.gen_dir, exist_ok=True)
        self.stats = {"tensors": 0, "changed_words": 0, "bytes": 0, "dense_bytes": 0}
        self._manifest: List[Dict[str, Any]] = []

    def send_bucket(self, bucket) -> List[Dict[str, Any]]:
        for name, t in bucket:
            cur = t.detach().cpu().contiguous()
            if cur.element_size() != 2:
                cur = cur.to(torch.bfloat16)
            prev = self.prev.get(name)
            entry = {"name": name, "shape": list(cur.shape), "dtype": str(cur.dtype).replace("torch.", "")}
            fname = name.replace("/", "_") + (".delta" if prev is not None else ".full")
            if prev is None:
                blob = cur.view(torch.uint8).numpy().tobytes() if cur.dtype != torch.bfloat16 \
                    else cur.view(torch.int16).numpy().tobytes()
                entry["kind"] = "full"
            else:
                blob = delta_encode(prev, cur)
                entry["kind"] = "delta"
                self.stats["changed_words"] += int.from_bytes(blob[8:16], "little")
            with open(os.path.join(self.gen_dir, fname), "wb") as f:
                f.write(blob)
            entry["file"] = fname
            self._manifest.append(entry)
            self.prev[name] = cur
            self.stats["tensors"] += 1
            self.stats["bytes"] += len(blob)
            self.stats["dense_bytes"] += cur.numel() * 2
        return self._manifest[-len(bucket):]

    def finish(self) -> str:
        p = os.path.join(self.gen_dir, "manifest.json")
        with open(p, "w") as f:
            json.dump({"generation": self.generation, "tensors": self._manifest, "stats": self.stats}, f)
        return p


def apply_delta_generation(gen_dir: str, weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    """Receiver side of ``SparseDeltaTransport``: updates ``weights`` in place / fills it."""
    with open(os.path.join(gen_dir, "manifest.json")) as f:
        man = json.load(f)
    for e in man["tensors"]:
        with open(os.path.join(gen_dir, e["file"]), "rb") as f:
            blob = f.read()
        if e["kind"] == "full":
            t = torch.frombuffer(bytearray(blob), dtype=torch.int16).view(getattr(torch, e["dtype"]))
            weights[e["name"]] = t.view(e["shape"]).clone()
        else:
            delta_apply(weights[e["name"]], blob)
    return weights


# ---------------------------------------------------------------------------------------------
# handler
# ---------------------------------------------------------------------------------------------
class WeightSyncHandler:
    """Drives one sync: pause engines -> stream buckets -> resume.  Lives on every trainer rank
    (the gathers are collective); only global rank 0 owns the transport."""

    def __init__(self, runner, endpoints: Optional[EndpointManager] = None):
        self.runner = runner
        self.endpoints = endpoints or EndpointManager()
        self.quantization: Optional[str] = None
        self.group: Optional[StatelessGroupBroadcaster] = None
        self.delta: Optional[SparseDeltaTransport] = None
        self.last: Dict[str, Any] = {}

    def _is_driver(self) -> bool:
        return (not dist.is_initialized()) or dist.get_rank() == 0

    def _ensure_group(self, master_addr: str, master_port: int, backend: str) -> StatelessGroupBroadcaster:
        if self.group is None:
            world = 1 + self.endpoints.total_world()
            self.endpoints.broadcast_post("/init_weights_update_group", lambda e, off: {
                "master_address": master_addr, "master_port": master_port, "rank_offset": off,
                "world_size": world, "group_name": "xorl_weight_sync", "backend": backend})
            self.group = StatelessGroupBroadcaster(master_addr, master_port, 0, world, backend,
                                                   self.runner.device)
        return self.group

    def sync(self, backend: str = "nccl_broadcast", quantization: Optional[str] = None,
             bucket_size_mb: int = 1024, directory: Optional[str] = None,
             master_addr: str = "127.0.0.1", master_port: int = 29600, transport=None,
             group_backend: Optional[str] = None, **_) -> Dict[str, Any]:
        r = self.runner
        quant = quantization or self.quantization
        driver = self._is_driver()
        t0 = time.time()
        out_dir = directory or os.path.join(r.output_dir, "sampler_weights", f"step_{r.step:06d}")
        if driver and transport is None:
            if backend == "file":
                transport = FileTransport(out_dir)
            elif backend == "sparse_delta":
                self.delta = self.delta or SparseDeltaTransport(directory or os.path.join(r.output_dir, "sampler_deltas"))
                self.delta.begin()
                transport = self.delta
            elif backend == "nccl_broadcast":
                gb = group_backend or ("nccl" if r.device.type == "cuda" else "gloo")
                transport = self._ensure_group(master_addr, master_port, gb)
            else:
                raise ValueError(f"backend {backend!r} needs an explicit transport")
        if driver and self.endpoints.endpoints:
            self.endpoints.broadcast_post("/pause_generation", lambda e, off: {})
        names, nbytes, nb = 0, 0, 0
        merged = None
        if getattr(r.model, "_xb_lora_config", None):
            # a LoRA policy is sent with its active adapter folded into the base weights
            from ..adapters.lora import merged_weight_view
            merged = merged_weight_view(r.engine)
        only, qcfg = None, None
        if getattr(r.model, "_xb_qarl_config", None):
            # a fake-quantised policy: the receiver gets exactly the wrapped weights, on the grid they trained on
            from ..adapters.qarl import sync_quantization_config
            qcfg = sync_quantization_config(r.model)
            trained = qcfg["quant_method"]
            fmt = getattr(r.trainer.args.train, "qarl_sync_format", trained)
            if quant not in (None, "bf16", trained):
                raise ValueError(f"sync quantization {quant!r} differs from the grid the policy trains on ({trained!r})")
            if quant != "bf16" and fmt != "bf16":
                quant, only = trained, set(qcfg["qarl"]["folded_modules"])
        stream = iter_sync_tensors(r.engine, r.model.config, torch.bfloat16, quant, merged, only)
        for bucket in bucketize(stream, bucket_size_mb << 20):
            if not driver:
                continue
            if isinstance(transport, StatelessGroupBroadcaster) and self.endpoints.endpoints:
                flat, manifest = flatten_bucket(bucket)
                self.endpoints.broadcast_post("/update_weights_from_distributed", lambda e, off: {
                    "names": [m["name"] for m in manifest], "dtypes": [m["dtype"] for m in manifest],
                    "shapes": [m["shape"] for m in manifest], "manifest": manifest,
                    "group_name": "xorl_weight_sync", "flush_cache": False})
                transport.broadcast(flat)
            else:
                transport.send_bucket(bucket)
            names += len(bucket)
            nbytes += sum(t.numel() * t.element_size() for _, t in bucket)
            nb += 1
        extra = {}
        if driver and hasattr(transport, "finish"):
            extra["index"] = transport.finish()
        if driver and isinstance(transport, SparseDeltaTransport):
            extra["delta_stats"] = dict(transport.stats)
        if driver and self.endpoints.endpoints:
            self.endpoints.broadcast_post("/continue_generation", lambda e, off: {})
        self.last = {"synced": True, "tensors": names, "bytes": nbytes, "buckets": nb,
                     "seconds": time.time() - t0, "backend": backend, "quantization": quant, **extra}
        if only is not None:
            self.last["quantization_config"] = qcfg
        return self.last
